"""flash_msa_b200: the Flash-MSA training hot path on B200 (sm_100a).

Public names are those of the reference package (flash_msa/__init__.py:3-14)."""
from .api import sparse_attention as flash_msa_func
from .api import sparse_attention_varlen as flash_msa_varlen_func
from .api import sparse_attention_warmup
from .api import sparse_attention_warmup_varlen as flash_msa_warmup_varlen_func
from .api import sparse_attention_warmup as flash_msa_func_warmup
from .api import sparse_attention_warmup as flash_msa_warmup_func
from .api import check_pending_status, last_kl_value

__all__ = [
    "flash_msa_func",
    "flash_msa_varlen_func",
    "flash_msa_warmup_varlen_func",
    "flash_msa_func_warmup",
    "flash_msa_warmup_func",
    "sparse_attention_warmup",
    "last_kl_value",
    "check_pending_status",
]
