"""`import corope_b200` -- an importable name for the package that lives in the directory `co-rope_b200/`.

A hyphen is not valid in a Python identifier, so the package directory itself can only be reached with
importlib.import_module("co-rope_b200").  This alias imports it that way and registers the package and its
submodules under the name `corope_b200` as well, so that

    import corope_b200
    from corope_b200 import fused_rope_attention, corope_gqa_attention, attention_fwd_bwd_host
    from corope_b200.fused_rope_attn import attention

all work and refer to the very same module objects (one loaded C-ABI library, one set of per-device state).
"""

import importlib
import sys

_real = importlib.import_module("co-rope_b200")
for _name, _mod in list(sys.modules.items()):
    if _name.startswith("co-rope_b200."):
        sys.modules[__name__ + _name[len("co-rope_b200"):]] = _mod
sys.modules[__name__] = _real
