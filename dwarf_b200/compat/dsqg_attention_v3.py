"""Import shim: `from dsqg_attention_v3 import ...` resolves to the B200 implementation
when this directory replaces the reference's kernels/ directory on sys.path."""
from dwarf_b200.modules import DSQGAttentionV3, dsqg_attention_v3  # noqa: F401
from dwarf_b200.ops import ALL_OFFSETS as _ALL

ALL_OFFSETS = list(_ALL)
