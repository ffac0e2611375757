"""The entry point that allocates nothing, called the way its users call it: through the
exported C symbol of the kernel library, with raw pointers.

Some hosts of the library cannot allocate device memory on the path that runs a decode step (a
latency-critical C++ loop that must not take the CUDA allocator's lock, or a process whose
device memory is already handed out in full).  For them ``gb_attention_decode_static`` merges the
key splits of single-token attention through an array inside the library image instead of
caller scratch.  Here it is compared with the ordinary entry point (``gb_attention_simt`` with
caller scratch) on two calls in a row of different shapes, so that what the first call leaves in
the shared array is seen not to matter.  The file sorts last so that a run that stops at the
first failure has already run every other test.
"""
import ctypes
import math
from ctypes import Structure, byref, c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Params(Structure):
    _fields_ = [("q", c_void_p), ("q_row_stride", c_int64), ("out", c_void_p), ("out_row_stride", c_int64),
                ("k_plane", c_void_p), ("v_plane", c_void_p), ("block_table", c_void_p), ("bt_stride", c_int),
                ("seq_slot", c_void_p), ("seq_q_start", c_void_p), ("seq_q_len", c_void_p),
                ("seq_kv_len", c_void_p), ("nseq", c_int), ("heads", c_int), ("kv_heads", c_int), ("d", c_int),
                ("max_q_len", c_int), ("scale", c_float), ("window", c_int), ("num_splits", c_int), ("scratch", c_void_p),
                ("pages", c_int), ("max_slots", c_int)]


@pytest.fixture(scope="module")
def lib():
    from gophonic_b200.csrc import build
    handle = ctypes.CDLL(build.ensure_built(verbose=False))
    handle.gb_last_error.restype = ctypes.c_char_p
    handle.gb_static_scratch_floats.restype = ctypes.c_uint
    return handle


def case(dtype, heads, kvh, d, kv_lens, splits, seed):
    g = torch.Generator().manual_seed(seed)
    nseq = len(kv_lens)
    max_pages = (max(kv_lens) + 63) // 64
    n_pages = nseq * max_pages + 2
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    table = perm[:nseq * max_pages].reshape(nseq, max_pages).contiguous().to(DEV)
    mk = lambda *s: torch.randn(*s, generator=g).to(device=DEV, dtype=dtype)
    k, v, q = mk(n_pages, kvh, 64, d), mk(n_pages, kvh, 64, d), mk(nseq, heads * d)
    ints = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    meta = dict(slot=ints(list(range(nseq))), start=ints(list(range(nseq))), qlen=ints([1] * nseq), kvlen=ints(kv_lens))
    out = torch.full((nseq, heads * d), float("nan"), dtype=dtype, device=DEV)
    p = Params(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k.data_ptr(), v.data_ptr(), table.data_ptr(),
               table.stride(0), meta["slot"].data_ptr(), meta["start"].data_ptr(), meta["qlen"].data_ptr(),
               meta["kvlen"].data_ptr(), nseq, heads, kvh, d, 1, 1.0 / math.sqrt(d), 0, splits, 0, n_pages, nseq)
    keep = (q, k, v, table, meta)
    return p, out, keep


def run_both(lib, dtype, heads, kvh, d, kv_lens, splits, seed):
    code = 0 if dtype == torch.float32 else 1
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    p, out_static, keep = case(dtype, heads, kvh, d, kv_lens, splits, seed)
    rc = lib.gb_attention_decode_static(byref(p), c_int(code), stream)
    assert rc == 0, lib.gb_last_error().decode()
    # the existing entry point, with scratch the caller allocates
    scratch = torch.empty(len(kv_lens) * heads * splits * (d + 2), dtype=torch.float32, device=DEV)
    out_ref = torch.full_like(out_static, float("nan"))
    p.out, p.scratch = out_ref.data_ptr(), scratch.data_ptr()
    rc = lib.gb_attention_simt(byref(p), c_int(code), stream)
    assert rc == 0, lib.gb_last_error().decode()
    torch.cuda.synchronize()
    assert torch.isfinite(out_static.float()).all()
    err = (out_static.double() - out_ref.double()).abs().max().item() / out_ref.double().abs().max().item()
    assert err < 1e-5, err
    return out_static


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_equals_the_ordinary_one_twice_in_a_row(lib, dtype):
    # first call: many long sequences, many splits, wide heads: fills much of the array
    run_both(lib, dtype, heads=8, kvh=2, d=128, kv_lens=[700, 64, 65, 333, 1, 500], splits=8, seed=1)
    # second call right after it, another shape: the array still holds the first call's partials
    run_both(lib, dtype, heads=6, kvh=3, d=32, kv_lens=[130, 2], splits=3, seed=2)


def test_static_scratch_entry_point_refuses_what_does_not_fit(lib):
    limit = lib.gb_static_scratch_floats()
    assert limit == 2 * 1024 * 1024
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    p, _, keep = case(torch.float32, 4, 2, 64, [100, 100], 4, 3)
    p.nseq = 4096  # 4096 * 4 * 4 * 66 floats: far beyond the array; refused before anything is read
    assert lib.gb_attention_decode_static(byref(p), c_int(0), stream) != 0
    assert b"exceed the static scratch" in lib.gb_last_error()
    p.nseq, p.num_splits = 2, 1
    assert lib.gb_attention_decode_static(byref(p), c_int(0), stream) != 0
    assert b"at least 2" in lib.gb_last_error()
    p.num_splits, p.max_q_len = 4, 3
    assert lib.gb_attention_decode_static(byref(p), c_int(0), stream) != 0
    assert b"single tokens" in lib.gb_last_error()
    torch.cuda.synchronize()
