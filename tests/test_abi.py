"""The C-ABI library loads on a host without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

import pytest

from megafold_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "megafold_b200.h")).read()
    return sorted(set(re.findall(r"MF_API[^;(]*?\b(mf_\w+)\s*\(", text)))


def test_header_symbols_all_bound_and_exported():
    names = _declared()
    assert len(names) >= 16
    assert sorted(_lib.SYMBOLS) == [n for n in names if n in _lib.SYMBOLS]
    handle = C.CDLL(_lib.LIB_PATH) if os.path.exists(_lib.LIB_PATH) else _lib.lib()
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
        assert n in _lib.SYMBOLS, f"{n} declared in the header but not bound in _lib.SYMBOLS"


def test_version_and_error_string():
    L = _lib.lib()
    assert L.mf_version() == 2
    assert isinstance(L.mf_last_error_string(), bytes)


def test_null_and_bad_args_are_rejected_without_a_gpu():
    L = _lib.lib()
    assert L.mf_evo_fwd(None, None) == -1
    a = _lib.EvoFwdArgs()
    assert L.mf_evo_fwd(C.byref(a), None) == -1          # sizes are zero
    assert b"positive" in L.mf_last_error_string()
    assert L.mf_swiglu_fwd(None, None, 4, 4, 0, None) == -1
    b = _lib.LnlBwdArgs()
    assert L.mf_lnl_bwd(C.byref(b), None) == -1
    assert L.mf_evo_bwd_workspace_bytes(None) == 0


def test_struct_layout_matches_c():
    # spot-check offsets that depend on padding rules (int32 block followed by pointers)
    assert _lib.EvoFwdArgs.q.offset == 40                 # 9 x int32 = 36 -> aligned to 8
    assert _lib.EvoBwdArgs.q.offset == 40                 # 10 x int32 = 40
    assert _lib.LnlFwdArgs.x.offset == 32                 # int64 + 4 x int32/float = 28 -> 32
    assert _lib.TransitionBwdArgs.x.offset == 24


def test_cpu_tensors_are_rejected():
    import torch
    import megafold_b200 as mfb
    q = torch.zeros(1, 2, 4, 1, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        mfb.TritonEvoformer(q, q, q, torch.ones(1, 2, 1, 1, 4, dtype=torch.bool), torch.zeros(1, 1, 1, 4, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        mfb.LayernormLinear(8, 4)(torch.zeros(3, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        mfb.FusedTransition(8)(torch.zeros(3, 8))
