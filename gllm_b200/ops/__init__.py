"""Hot-path ops. CUDA tensors run the hand-written sm_100a kernels; CPU tensors run the fp32 oracle."""
from . import _native
from .attention import DecodeWorkspace, attention_ref, paged_decode, paged_prefill
from .elementwise import (argmax, embed_gather, glu, layernorm, pool, rmsnorm, rope_kv_write, sample,
                          sample_ref, filtered_probs_ref)
from .linear import (ACT_IDS, gemm, gemm_fp8, gemm_glu, gemm_grouped, gemm_qkv, gemm_residual, set_pair_max_m, set_pair_big_m,
                     interleave_gate_up, deinterleave_gate_up, pad_rows, rope_ref)
