"""Host-side metadata of the fused prefill path (same export list as the reference
``src/mega_attention/metadata/__init__.py:3-31``, plus the names the reference keeps
module-private but its tests and workspace import directly)."""
from .row_desc import (
    AR_M_TILE,
    FA_M_TILE,
    OPROJ_M_TILE,
    ROW_M_TILE,
    RowDescMeta,
    active_counts,
    build_row_desc,
    cdiv,
    csym_numel,
    cu_seqlens_from_seqlens,
    decode_oproj_slot,
    oproj_task_counts,
    oscratch_numel,
)
from .launch_heuristic import LaunchConfig, choose_launch_config, estimate_work_ratio

__all__ = [
    "AR_M_TILE", "FA_M_TILE", "OPROJ_M_TILE", "ROW_M_TILE", "RowDescMeta",
    "build_row_desc", "cdiv", "csym_numel", "cu_seqlens_from_seqlens",
    "decode_oproj_slot", "oproj_task_counts", "oscratch_numel",
    "active_counts", "LaunchConfig", "choose_launch_config", "estimate_work_ratio",
]
