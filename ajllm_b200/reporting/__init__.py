"""Model reports and resource estimates."""

from ajllm_b200.reporting.model_report import write_model_report
from ajllm_b200.reporting.resource_estimates import ResourceEstimate, estimate_resources

__all__ = ["write_model_report", "ResourceEstimate", "estimate_resources"]
