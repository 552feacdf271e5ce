"""Runtime helpers: device choice, seeding, device-side timing, clock sampling."""

from ajllm_b200.utils.device import describe_device_choice, pick_device
from ajllm_b200.utils.seeding import seed_all

# the reference's names for the same functions (``ajllm/utils/device.py:8-25``, ``ajllm/utils/random.py:11``)
resolve_device = pick_device
explain_device_selection = describe_device_choice
seed_everything = seed_all

__all__ = ["pick_device", "describe_device_choice", "seed_all", "resolve_device", "explain_device_selection",
           "seed_everything"]
