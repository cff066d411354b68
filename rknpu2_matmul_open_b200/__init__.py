"""B200-native W4A8 quantized linear: Python host mirror of the C ABI in ``include/``."""
from . import capi  # noqa: F401
from .w4a8 import (Context, Domain, W4A8Error, Weights, Workspace, default_config, enqueue_batch_f16, enqueue_ffn_f32,  # noqa: F401
                   memory_query, run_ffn_f32)
from . import w8a8  # noqa: F401
from . import moe  # noqa: F401
