"""Runtime helpers: device choice, seeding, device-side timing, clock sampling."""

from ajllm_b200.utils.device import describe_device_choice, pick_device
from ajllm_b200.utils.seeding import seed_all

__all__ = ["pick_device", "describe_device_choice", "seed_all"]
