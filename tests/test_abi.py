"""CPU: the C-ABI library builds, loads, exports what include/evoattn.h declares, keeps the
struct layout the header declares, and rejects bad requests before touching a GPU."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "evoattn.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(evoattn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_library):
    lib = C.CDLL(built_library)
    names = declared_symbols()
    assert "evoattn_fwd" in names and "evoattn_bwd" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in evoattn.h but not exported"


def test_python_binding_lists_the_same_symbols(built_library):
    from evoformer_triton_b200 import _lib
    assert sorted(_lib.SYMBOLS) == declared_symbols()
    assert _lib.load().evoattn_abi_version() == _lib.ABI_VERSION


def test_struct_layout_matches_header(built_library, tmp_path):
    from evoformer_triton_b200 import _lib
    src = tmp_path / "sz.c"
    src.write_text('#include "evoattn.h"\n#include <stdio.h>\n#include <stddef.h>\n'
                   'int main(){printf("%zu %zu %zu %zu %zu\\n", sizeof(evoattn_fwd_params),'
                   'sizeof(evoattn_bwd_params), offsetof(evoattn_fwd_params, mask),'
                   'offsetof(evoattn_fwd_params, status), offsetof(evoattn_bwd_params, workspace));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(_lib.FwdParams), C.sizeof(_lib.BwdParams), _lib.FwdParams.mask.offset,
            _lib.FwdParams.status.offset, _lib.BwdParams.workspace.offset]
    assert got == want


def test_bad_requests_are_rejected_without_a_gpu(built_library):
    from evoformer_triton_b200 import _lib
    lib = _lib.load()
    p = _lib.FwdParams()
    assert lib.evoattn_fwd(None, None) == 1            # null params
    assert lib.evoattn_fwd(C.byref(p), None) == 1      # null tensors
    p.q = p.k = p.v = p.o = p.lse = 256                # fake non-null addresses: never dereferenced
    p.dtype = 7
    assert lib.evoattn_fwd(C.byref(p), None) == 3      # dtype
    p.dtype = _lib.BF16
    assert lib.evoattn_fwd(C.byref(p), None) == 2      # zero dims
    p.B = p.H = p.S = p.R = 1
    p.D = 256
    assert lib.evoattn_fwd(C.byref(p), None) == 5      # D > 128
    p.D = 32
    p.mask_kind = _lib.MASK_BOOL
    assert lib.evoattn_fwd(C.byref(p), None) == 1      # mask kind without a mask
    b = _lib.BwdParams()
    b.fwd = p
    b.fwd.mask_kind = 0
    assert lib.evoattn_bwd(C.byref(b), None) == 1      # null gradients
    assert lib.evoattn_bwd_workspace_bytes(C.byref(b)) == 0
    # the in-call exchange of d(pair_bias) must work on the caller's own exchange buffer
    b.d_o = b.dq = b.dk = b.dv = 256
    x = _lib.PeerAllReduceParams()
    x.world, x.rank, x.count = 2, 0, 1
    bufs = (C.c_void_p * 2)(512, 768)
    x.bufs = bufs
    b.exchange = C.pointer(x)
    assert lib.evoattn_bwd(C.byref(b), None) == 1      # an exchange without a bias and its gradient
    b.fwd.bias = 1024
    b.dbias = 4096
    assert lib.evoattn_bwd(C.byref(b), None) == 2      # dbias is not this rank's exchange buffer
    b.dbias = 512
    x.count = 7
    assert lib.evoattn_bwd(C.byref(b), None) == 2      # count is not B*H*R*R
    assert "null" in _lib.strerror(1)
    assert _lib.strerror(12345) == "unknown status"


def test_op_refuses_cpu_tensors(built_library):
    import torch
    from evoformer_triton_b200 import EvoformerAttention
    q = torch.zeros(1, 1, 8, 1, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        EvoformerAttention.apply(q, q, q, None, None)


def test_missing_library_fails_loudly(monkeypatch):
    from evoformer_triton_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libevoattn.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
