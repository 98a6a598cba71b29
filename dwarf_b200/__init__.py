"""dwarf_b200: B200-native (sm_100a) DSQG attention -- forward, backward and ring-buffer
decode as hand-written CUDA behind a C ABI (include/dsqg_b200.h), with the DWARF
reference's Python operator interface on top."""
from .ops import (ALL_OFFSETS, OFFSETS_43, OFFSETS_45, SPARSE_TAPS, DSQGFunction, DSQGPackedFunction,
                  dsqg_attention, dsqg_attention_packed, dsqg_forward_lse, packed_path_available)
from .modules import (DSQGAttentionN_Fused, DSQGAttentionQW, DSQGAttentionV3, dsqg_attention_v2,
                      dsqg_attention_v3)
from .decode import DSQGRingCache, dsqg_decode_step
from .host import DSQGHostPipeline
from ._lib import DSQGError

__all__ = ["ALL_OFFSETS", "OFFSETS_43", "OFFSETS_45", "SPARSE_TAPS", "DSQGFunction", "dsqg_attention",
           "dsqg_forward_lse", "DSQGPackedFunction", "dsqg_attention_packed", "packed_path_available", "DSQGAttentionN_Fused", "DSQGAttentionQW", "DSQGAttentionV3",
           "dsqg_attention_v2", "dsqg_attention_v3", "DSQGRingCache", "dsqg_decode_step", "DSQGHostPipeline", "DSQGError"]
