"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of this library may not allocate device memory where they call it: under another
framework's allocator, inside a real-time loop, in a plugin that must not allocate after
start-up.  `ri_attention_decode_static` keeps the scratch for the split partial results in a
fixed device array inside the library instead of asking the caller for it.  Here it is
called twice in a row, on different inputs, and must give what the regular entry point
(which is handed scratch tensors) gives.  This file is collected last on purpose: if it
fails, a run that stops at the first failure has already run everything else.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(seed, n_seqs, nh, nkv, hd, lengths):
    """A scrambled paged cache holding `lengths[b]` keys per sequence, and one query row each."""
    g = torch.Generator().manual_seed(seed)
    page = 64
    pages_per = [-(-n // page) for n in lengths]
    n_pages = sum(pages_per) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(n_seqs, max(pages_per) + 1, dtype=torch.int32)
    i = 0
    for b, n in enumerate(pages_per):
        for pg in range(n):
            table[b, pg] = perm[i]
            i += 1
    kc = torch.randn(n_pages, nkv, page, hd, generator=g).bfloat16()
    vc = torch.randn(n_pages, nkv, page, hd, generator=g).bfloat16()
    q = torch.randn(n_seqs, (nh + 2 * nkv) * hd, generator=g).bfloat16()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return dict(q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), table=table.to(DEV), slot=i32(list(range(n_seqs))),
                length=i32(lengths), cu=i32(list(range(n_seqs + 1))))


def _p(t):
    return c_void_p(t.data_ptr())


def test_static_scratch_entry_point_matches_the_regular_one():
    from rust_inference_b200.kernels import ops
    from rust_inference_b200.kernels.build import load
    lib = load("attention_mma")
    fn = lib.ri_attention_decode_static
    fn.restype = c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    # two calls in a row with different shapes: the second reuses the array the first one left dirty
    for seed, (n_seqs, nh, nkv, hd, lengths, splits) in enumerate([
            (3, 28, 4, 128, [1000, 64, 129], 8),
            (5, 8, 2, 64, [1, 700, 63, 65, 300], 3)]):
        c = _case(seed, n_seqs, nh, nkv, hd, lengths)
        scale = hd ** -0.5
        want = torch.zeros(n_seqs, nh * hd, device=DEV, dtype=torch.bfloat16)
        po = torch.zeros(n_seqs * nh * splits * hd, device=DEV)
        pml = torch.zeros(n_seqs * nh * splits * 2, device=DEV)
        ops.attention_decode(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["slot"], c["length"], c["cu"],
                             want, n_seqs=n_seqs, n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=64,
                             scale=scale, window=0, n_splits=splits, part_o=po, part_ml=pml)
        got = torch.zeros_like(want)
        rc = fn(_p(c["q"]), c_int(c["q"].shape[1]), _p(c["kc"]), _p(c["vc"]), _p(c["table"]),
                c_int(c["table"].shape[1]), _p(c["slot"]), _p(c["length"]), _p(c["cu"]), _p(got),
                c_int(got.shape[1]), c_int(n_seqs), c_int(nh), c_int(nkv), c_int(hd), c_int(64), c_float(scale),
                c_int(0), c_int(splits), stream)
        assert rc == 0, lib.ri_last_error().decode()
        torch.cuda.synchronize()
        # same kernels, same inputs, same split: the results are equal, well inside the 2e-2 the
        # attention tests allow
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2e-2 * want.float().abs().max().item(), err
        assert torch.equal(got, want)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from rust_inference_b200.kernels.build import load
    lib = load("attention_mma")
    fn = lib.ri_attention_decode_static
    fn.restype = c_int
    c = _case(0, 2, 4, 2, 64, [10, 20])
    out = torch.zeros(2, 4 * 64, device=DEV, dtype=torch.bfloat16)
    # 4096 sequences x 64 heads x 32 splits x 130 floats is far beyond the 2 Mi floats of the array
    rc = fn(_p(c["q"]), c_int(c["q"].shape[1]), _p(c["kc"]), _p(c["vc"]), _p(c["table"]), c_int(c["table"].shape[1]),
            _p(c["slot"]), _p(c["length"]), _p(c["cu"]), _p(out), c_int(out.shape[1]), c_int(4096), c_int(64),
            c_int(2), c_int(128), c_int(64), c_float(0.1), c_int(0), c_int(32),
            c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    msg = lib.ri_last_error().decode()
    assert "exceed the built-in scratch" in msg
    torch.cuda.synchronize()
