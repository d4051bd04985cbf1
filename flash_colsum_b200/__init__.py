"""flash_colsum for B200: attention column means with hand-written sm_100a kernels."""

from .ops import (flash_colsum, flash_colsum_causal, flash_colsum_host, topk_columns, threshold_columns,
                  device_status)

__all__ = ["flash_colsum", "flash_colsum_causal", "flash_colsum_host", "topk_columns", "threshold_columns",
           "device_status"]

__version__ = "0.2.2"
