"""Stand-alone, non-invasive tools: each entry point measures an optimizer in a short dry run
(restoring weights and state afterwards) or reports a recommendation the caller may apply."""
from .lr_calibration import (GroupUpdateStats, LRRangeResult, ParamVsAdamw, RelativeCalibration,
                             calibrate_relative, calibrate_vs_adamw, lr_range_test, measure_update_rms)

__all__ = ["GroupUpdateStats", "RelativeCalibration", "ParamVsAdamw", "LRRangeResult",
           "measure_update_rms", "calibrate_relative", "calibrate_vs_adamw", "lr_range_test"]
