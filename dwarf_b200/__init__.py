"""dwarf_b200: B200-native (sm_100a) DSQG attention -- forward, backward and ring-buffer
decode as hand-written CUDA behind a C ABI (include/dsqg_b200.h), with the DWARF
reference's Python operator interface on top."""
from .ops import (ALL_OFFSETS, causal_mean, OFFSETS_43, OFFSETS_45, SPARSE_TAPS, DSQGFunction, DSQGPackedFunction,
                  dsqg_attention, dsqg_attention_packed, dsqg_forward_lse, packed_path_available)
from .modules import (InterferenceInjection, DSQGAttentionN_Fused, DSQGAttentionQW, DSQGAttentionV3, dsqg_attention_v2,
                      dsqg_attention_v3)
from .decode import DSQGRingCache, dsqg_decode_step, dsqg_decode_step_kv
from .host import DSQGHostPipeline
from ._lib import DSQGError

__all__ = ["ALL_OFFSETS", "OFFSETS_43", "OFFSETS_45", "SPARSE_TAPS", "DSQGFunction", "dsqg_attention",
           "dsqg_forward_lse", "causal_mean", "DSQGPackedFunction", "dsqg_attention_packed", "packed_path_available", "DSQGAttentionN_Fused", "InterferenceInjection", "DSQGAttentionQW", "DSQGAttentionV3",
           "dsqg_attention_v2", "dsqg_attention_v3", "DSQGRingCache", "dsqg_decode_step", "dsqg_decode_step_kv", "DSQGHostPipeline", "DSQGError"]
