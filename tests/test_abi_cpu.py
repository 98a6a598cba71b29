"""CPU tests of the C-ABI boundary: the library loads, exports every declared symbol, and
rejects bad arguments on the host with a status code (no kernel is launched, no GPU needed)."""
import ctypes
import os
import re

import pytest

from dwarf_b200 import _lib
from dwarf_b200.build import build_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "dsqg_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsqg_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_functions()
    assert {"dsqg_fwd", "dsqg_bwd", "dsqg_decode", "dsqg_bwd_scratch_bytes", "dsqg_status_str"} <= set(names)
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/dsqg_b200.h but not exported"
    assert set(names) == set(_lib.EXPORTED_SYMBOLS)


def test_status_strings(lib):
    assert lib.dsqg_status_str(0) == b"ok"
    for code in range(-9, 0):
        assert len(lib.dsqg_status_str(code)) > 3
    assert lib.dsqg_status_str(-99) == b"unknown status"
    assert lib.dsqg_version() >= 100


def _fake(n=1):
    return 4096 * n      # a non-null, 16-byte aligned fake device address (never dereferenced)


def _off(vals):
    return (ctypes.c_int32 * len(vals))(*vals), len(vals)


def call_fwd(lib, q=_fake(1), k=_fake(2), v=_fake(3), pb=_fake(4), se=None, hg=None,
             offsets=(0, 1, 2, 8), out=_fake(5), lse=_fake(6), B=1, H=2, N=16, D=32, dtype=0):
    off, J = _off(offsets) if offsets is not None else (None, 4)
    return lib.dsqg_fwd(q, k, v, pb, se, hg, off, J, out, lse, B, H, N, D, dtype, None)


def test_fwd_argument_errors_are_statuses(lib):
    assert call_fwd(lib, q=None) == -1
    assert call_fwd(lib, lse=None) == -1
    assert call_fwd(lib, offsets=None) == -1
    assert call_fwd(lib, D=33) == -2 and call_fwd(lib, D=0) == -2 and call_fwd(lib, D=136) == -2
    assert call_fwd(lib, N=0) == -2 and call_fwd(lib, B=-1) == -2
    assert call_fwd(lib, B=32768, H=2) == -2          # one grid row per (batch, head): B*H <= 65535
    assert call_fwd(lib, offsets=(0, 2, 2)) == -3 and call_fwd(lib, offsets=(-1, 0)) == -3
    assert call_fwd(lib, offsets=(3, 1)) == -3
    assert call_fwd(lib, offsets=tuple(range(129))) == -2
    assert call_fwd(lib, dtype=7) == -4
    assert call_fwd(lib, q=_fake(1) + 8) == -5 and call_fwd(lib, out=_fake(5) + 2) == -5


def test_bwd_scratch_and_argument_errors(lib):
    n = lib.dsqg_bwd_scratch_bytes(43, 32, 8, 2048, 32, 0)
    assert n >= 32 * 8 * 2048 * 4
    assert lib.dsqg_bwd_scratch_bytes(43, 32, 8, 2048, 32, 1) > n
    assert lib.dsqg_bwd_scratch_bytes(0, 1, 1, 1, 32, 0) == 0
    assert lib.dsqg_bwd_scratch_bytes(43, 1, 1, 16, 12, 0) == 0
    off, J = _off((0, 1, 4))
    args = dict(B=1, H=1, N=16, D=32)
    need = lib.dsqg_bwd_scratch_bytes(J, 1, 1, 16, 32, 0)

    def call(scratch=_fake(20), nbytes=need, dq=_fake(10), hg=None, dhg=None, dtype=0):
        return lib.dsqg_bwd(_fake(1), _fake(2), _fake(3), _fake(4), None, hg, off, J,
                            _fake(5), _fake(6), _fake(7), dq, _fake(11), _fake(12),
                            _fake(13), None, dhg, scratch, nbytes, 1, 1, 16, 32, dtype, None)
    assert call(nbytes=need - 1) == -6
    assert call(scratch=None) == -1 and call(dq=None) == -1
    assert call(hg=_fake(30), dhg=None) == -1          # gain given but no place for its gradient
    assert call(scratch=_fake(20) + 4) == -5
    assert call(dtype=2) == -4


def test_decode_argument_errors(lib):
    off, J = _off((0, 1, 2, 5))

    for entry in (lib.dsqg_decode, lib.dsqg_decode_overlapped):      # same checks, no launch
        def call(R=6, head=_fake(8), S=2, D=64, kr=_fake(4)):
            return entry(_fake(1), _fake(2), _fake(3), kr, _fake(5), head, None,
                         _fake(6), None, None, off, J, R, _fake(7), S, 2, D, 0, None)
        assert call(R=5) == -3                  # max offset must be < R
        assert call(head=None) == -1
        assert call(D=12) == -2 and call(S=0) == -2
        assert call(kr=_fake(4) + 8) == -5


def test_ring_prefill_argument_errors(lib):
    call = lambda **kw: lib.dsqg_ring_prefill(kw.get("k", _fake(1)), _fake(2), _fake(3), _fake(4), _fake(5),
                                              kw.get("fill", _fake(6)), 2, 2, kw.get("N", 8), kw.get("D", 64), kw.get("R", 16), 0, None)
    assert call(k=None) == -1 and call(fill=None) == -1
    assert call(N=0) == -2 and call(D=12) == -2 and call(R=0) == -2
    assert call(k=_fake(1) + 4) == -5


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    from dwarf_b200 import dsqg_attention
    q = torch.zeros(1, 1, 8, 32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        dsqg_attention(q, q, q, torch.zeros(44, 1))


def test_kernel_path_knob(lib):
    assert lib.dsqg_set_kernel_path(1) == 0 and lib.dsqg_set_kernel_path(0) == 0
    assert lib.dsqg_set_kernel_path(2) == 0 and lib.dsqg_set_kernel_path(3) == 0 and lib.dsqg_set_kernel_path(4) == 0
    assert lib.dsqg_set_kernel_path(0) == 0
    assert lib.dsqg_set_kernel_path(5) == -8


def test_tensor_core_path_query_and_scaled_entry_checks(lib):
    j43 = tuple(range(32)) + (48, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536)
    j44 = tuple(range(33)) + j43[32:]
    q = lambda dtype, D, offs, se: lib.dsqg_tensor_core_path(dtype, D, *_off(offs), se)
    assert q(0, 32, j43, 0) == 1 and q(0, 64, j44, 1) == 1 and q(0, 96, j43, 0) == 1 and q(0, 128, j43, 0) == 1
    assert q(0, 80, j43, 0) == 0 and q(0, 48, j43, 0) == 0          # odd widths: CUDA-core kernels unless padded
    d41 = tuple(range(41)) + (128, 384, 1536)
    assert q(0, 96, j44, 0) == 1 and q(0, 64, d41, 0) == 1
    assert q(0, 96, j43, 1) == 0 and q(0, 96, d41, 0) == 0          # wide heads: dense window up to 32, no scale_embed
    assert q(1, 32, j43, 0) == 0                                    # fp32 storage
    assert q(0, 32, (3, 1), 0) == 0 and q(0, 33, j43, 0) == 0       # invalid arguments
    off, J = _off((0, 1, 2, 8))
    fwd = lambda scale: lib.dsqg_fwd_scaled(_fake(1), _fake(2), _fake(3), _fake(4), None, None, off, J,
                                            _fake(5), _fake(6), 1, 2, 16, 32, 0, None, scale)
    assert fwd(0.0) == -8 and fwd(-1.0) == -8 and fwd(float("inf")) == -8 and fwd(float("nan")) == -8
    bwd = lambda scale: lib.dsqg_bwd_scaled(_fake(1), _fake(2), _fake(3), _fake(4), None, None, off, J,
                                            _fake(5), _fake(6), _fake(7), _fake(10), _fake(11), _fake(12),
                                            _fake(13), None, None, _fake(20), 1 << 20, 1, 1, 16, 32, 0, None, scale)
    assert bwd(0.0) == -8 and bwd(float("nan")) == -8


def test_strided_gate_scan_and_interleaved_ring_argument_errors(lib):
    """The entries added for caller layouts, the gate backward, the causal mean and the one-ring decode:
    every bad argument is a status on the host, nothing is launched."""
    off, J = _off((0, 1, 2, 8))
    good = _lib.Strides(3 * 2 * 32 * 16, 32, 3 * 2 * 32)
    odd = _lib.Strides(3 * 2 * 32 * 16, 32, 3 * 2 * 32 + 4)           # not a multiple of 8 elements
    neg = _lib.Strides(-8, 32, 192)

    def fwd(st_in=good, st_out=good, q=_fake(1), D=32, dtype=0, gate=None, scale=0.0):
        return lib.dsqg_fwd_strided(q, _fake(2), _fake(3), st_in, _fake(4), None, off, J, _fake(5), st_out, gate,
                                    _fake(6), 1, 2, 16, D, dtype, None, scale)
    assert fwd(st_in=None) == -1 and fwd(st_out=None) == -1 and fwd(q=None) == -1
    assert fwd(st_in=odd) == -5 and fwd(st_out=neg) == -5 and fwd(gate=_fake(9) + 2) == -5
    assert fwd(D=80) == -8 and fwd(dtype=1) == -8 and fwd(D=12) == -2
    assert fwd(scale=float("inf")) == -8

    need = lib.dsqg_bwd_scratch_bytes(J, 1, 2, 16, 32, 0)

    def bwd(st_in=good, st_out=good, scratch=_fake(20), nbytes=need, D=32, dq=_fake(10)):
        return lib.dsqg_bwd_strided(_fake(1), _fake(2), _fake(3), st_in, _fake(4), None, off, J, _fake(5), _fake(6),
                                    _fake(7), st_out, None, dq, _fake(11), _fake(12), _fake(13), None,
                                    scratch, nbytes, 1, 2, 16, D, 0, None, 0.0)
    assert bwd(st_in=None) == -1 and bwd(dq=None) == -1 and bwd(scratch=None) == -1
    assert bwd(st_out=odd) == -5 and bwd(nbytes=need - 1) == -6 and bwd(D=80) == -8

    # the scale_embed variants: the table is required, head widths above 64 have no kernel, and the
    # backward wants the larger scratch
    def fwd_se(se=_fake(8), D=32, st_in=good):
        return lib.dsqg_fwd_strided_se(_fake(1), _fake(2), _fake(3), st_in, _fake(4), se, None, off, J, _fake(5), good,
                                       None, _fake(6), 1, 2, 16, D, 0, None, 0.0)
    assert fwd_se(se=None) == -1 and fwd_se(se=_fake(8) + 4) == -5 and fwd_se(D=128) == -8 and fwd_se(st_in=odd) == -5
    need_se = lib.dsqg_bwd_scratch_bytes(J, 1, 2, 16, 32, 1)

    def bwd_se(se=_fake(8), dse=_fake(14), nbytes=need_se, D=32):
        return lib.dsqg_bwd_strided_se(_fake(1), _fake(2), _fake(3), good, _fake(4), se, None, off, J, _fake(5),
                                       _fake(6), _fake(7), good, None, _fake(10), _fake(11), _fake(12), _fake(13),
                                       dse, None, _fake(20), nbytes, 1, 2, 16, D, 0, None, 0.0)
    assert bwd_se(se=None) == -1 and bwd_se(dse=None) == -1 and bwd_se(D=128, nbytes=1 << 30) == -8
    assert need_se > need and bwd_se(nbytes=need) == -6

    gate = lambda **kw: lib.dsqg_gate_bwd(kw.get("dy", _fake(1)), _fake(2), _fake(3), kw.get("st", good), _fake(4),
                                          _fake(5), kw.get("delta", _fake(6)), 1, 2, 16, kw.get("D", 32), None)
    assert gate(dy=None) == -1 and gate(st=None) == -1 and gate(delta=None) == -1
    assert gate(st=odd) == -5 and gate(dy=_fake(1) + 8) == -5 and gate(D=12) == -2

    mean = lambda **kw: lib.dsqg_causal_mean(kw.get("x", _fake(1)), kw.get("out", _fake(2)), kw.get("B", 2), kw.get("N", 16),
                                             kw.get("D", 64), kw.get("dtype", 0), 0, None)
    assert mean(x=None) == -1 and mean(out=None) == -1 and mean(dtype=3) == -4
    assert mean(D=12) == -2 and mean(N=0) == -2 and mean(B=70000) == -2 and mean(x=_fake(1) + 4) == -5

    off4, J4 = _off((0, 1, 2, 5))
    dec = lambda **kw: lib.dsqg_decode_kv(_fake(1), _fake(2), _fake(3), kw.get("kv", _fake(4)), kw.get("head", _fake(8)), None,
                                          _fake(6), None, None, off4, J4, kw.get("R", 6), _fake(7), kw.get("S", 2), 2,
                                          kw.get("D", 64), 0, None, 0)
    assert dec(kv=None) == -1 and dec(head=None) == -1 and dec(R=5) == -3 and dec(D=12) == -2 and dec(S=0) == -2
    assert dec(kv=_fake(4) + 8) == -5
    pre = lambda **kw: lib.dsqg_ring_prefill_kv(kw.get("k", _fake(1)), _fake(2), kw.get("kv", _fake(3)), _fake(5), _fake(6),
                                                2, 2, kw.get("N", 8), kw.get("D", 64), kw.get("R", 16), 0, None)
    assert pre(k=None) == -1 and pre(kv=None) == -1 and pre(N=0) == -2 and pre(R=0) == -2 and pre(kv=_fake(3) + 4) == -5
    assert lib.dsqg_test_wait_timeout(0, None) == -8 and lib.dsqg_test_wait_timeout(3 * 10 ** 9, None) == -8
