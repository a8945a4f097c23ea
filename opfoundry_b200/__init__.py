"""B200 (sm_100a) sparse-MLA attention: hand-written CUDA kernels behind a C ABI, with a thin
host-side mirror of the reference launcher interface.  There is no CPU or PyTorch fallback."""
from . import api, synth  # noqa: F401
from .api import (mla_decode_plan_create, mla_decode_launch_pipeline, sparse_mla_prefill, debug_rows,  # noqa: F401
                  pack_fp8_rows, plan_host, lib)
