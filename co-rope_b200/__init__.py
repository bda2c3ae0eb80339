"""corope_b200: B200 (sm_100a) kernels for fused-RoPE attention and Co-RoPE GQA attention behind the
reference's Python entry points.  The directory name carries a hyphen; import it with
`importlib.import_module("co-rope_b200")`, or put the directory on sys.path and import
`fused_rope_attn` / `flash_attn_co_rope_gqa_triton` by the reference's own module names."""

from . import _ext  # noqa: F401
from .fused_rope_attn import attention as fused_rope_attention  # noqa: F401
from .fused_rope_attn import attention_theta as fused_rope_attention_theta  # noqa: F401
from .flash_attn_v2_triton import attention as flash_attention  # noqa: F401
from .flash_attn_co_rope_gqa_triton import attention as corope_gqa_attention  # noqa: F401
from .sharding import shard_units, unit_range  # noqa: F401
from .host_pipeline import attention_fwd_bwd_host  # noqa: F401
from ._ext import build, check_status  # noqa: F401
