"""Each kernel alone against a plain float32 reference of the same operation, at sizes other
than the engine tests use (odd widths, head sizes in steps of 16, many heads and groups)."""
import math

import pytest
import torch

import plain_impl
from rust_inference_b200.sampling import rng

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    from rust_inference_b200.kernels import ops
    return ops


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [7, 64, 1000, 3584])
def test_embed_gather(dtype, hidden):
    ops = _ops()
    table = torch.randn(50, hidden, device=DEV).to(dtype)
    ids = torch.tensor([0, 49, 7, 7, 13], dtype=torch.int32, device=DEV)
    out = torch.empty(5, hidden, device=DEV)
    ops.embed_gather(table, ids, out)
    assert torch.equal(out, plain_impl.embedding(table.float(), ids.tolist()))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, eps", [(5, 1e-5), (144, 1e-6), (1000, 1e-3), (3584, 1e-6), (5120, 1e-5)])
def test_rmsnorm(out_dtype, n, eps):
    ops = _ops()
    x = torch.randn(9, n, device=DEV) * 3
    x[3] *= 1e-3                                     # a row where eps matters
    w = torch.randn(n, device=DEV)
    out = torch.empty(9, n, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w, eps, out)
    want = plain_impl.rmsnorm(x.double().cpu(), w.double().cpu(), eps)
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    assert ((out.double().cpu() - want).abs() <= tol * want.abs().clamp_min(1e-3)).all()
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, n, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w, eps, picked, rows)
    assert torch.equal(picked, out[[8, 0, 3]])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_rows, n", [(300, 144), (257, 1000), (2048, 3584), (260, 5120), (256, 8192)])
def test_rmsnorm_of_many_rows(out_dtype, n_rows, n):
    """Steps of many rows take a kernel with one warp per row (and any width it cannot hold, another)."""
    ops = _ops()
    x = torch.randn(n_rows, n, device=DEV) * 2
    x[7] *= 1e-3
    w = torch.randn(n, device=DEV)
    out = torch.empty(n_rows, n, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w, 1e-6, out)
    pick = [0, 7, n_rows // 2, n_rows - 1]
    want = plain_impl.rmsnorm(x[pick].double().cpu(), w.double().cpu(), 1e-6)
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    assert ((out[pick].double().cpu() - want).abs() <= tol * want.abs().clamp_min(1e-3)).all()
    # every row as the few-rows kernel computes it
    few = torch.empty(8, n, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x[100:108].contiguous(), w, 1e-6, few)
    assert (out[100:108].double() - few.double()).abs().max().item() <= tol * few.double().abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [11, 176, 18944])
def test_silu_mul(dtype, inter):
    ops = _ops()
    gu = (torch.randn(5, 2 * inter, device=DEV) * 4).to(dtype)
    out = torch.empty(5, inter, device=DEV, dtype=dtype)
    ops.silu_mul(gu, out)
    g = gu.float().cpu()
    want = plain_impl.silu(g[:, :inter]) * g[:, inter:]
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert torch.allclose(out.float().cpu(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("style", ["half", "interleaved"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, hd", [(3, 1, 6), (8, 2, 16), (5, 5, 48), (28, 4, 128)])
def test_rope_and_cache_write(style, dtype, nh, nkv, hd):
    """Rotation against the plain table and rotation; keys and values must land at the page and
    offset of their position, with pages handed out in a scrambled order."""
    ops = _ops()
    from rust_inference_b200.parts.rope import rope_tables
    page, n_pages, base = 64, 9, 500000.0
    starts, news = [0, 100, 63], [70, 1, 2]
    cos, sin = rope_tables(hd, base, 256)
    pcos, psin = plain_impl.rope_table(hd, base, 256)
    assert torch.equal(torch.from_numpy(cos), pcos) and torch.equal(torch.from_numpy(sin), psin)
    table = torch.tensor([[5, 2, 0], [7, 1, 0], [3, 8, 0]], dtype=torch.int32)       # [slot][logical page]
    slots = [2, 0, 1]
    T = sum(news)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd).to(dtype)
    token_pos = torch.tensor([s + i for s, n in zip(starts, news) for i in range(n)], dtype=torch.int32)
    token_seq = torch.tensor([b for b, n in enumerate(news) for _ in range(n)], dtype=torch.int32)
    kc = torch.full((n_pages, nkv, page, hd), 77.0).to(dtype)
    vc = torch.full((n_pages, nkv, page, hd), 77.0).to(dtype)
    d = lambda t: t.to(DEV)
    q_dev, kc_dev, vc_dev = d(qkv.clone()), d(kc), d(vc)
    ops.rope_cache_write(q_dev, d(torch.from_numpy(cos)), d(torch.from_numpy(sin)), d(token_pos), d(token_seq),
                         d(torch.tensor(slots, dtype=torch.int32)), d(table), kc_dev, vc_dev, n_heads=nh,
                         n_kv_heads=nkv, head_dim=hd, page_size=page, style={"half": 0, "interleaved": 1}[style],
                         write_kv=True)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    x = qkv.float()
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for t in range(T):
        pos, b = int(token_pos[t]), int(token_seq[t])
        c, s_ = pcos[pos:pos + 1], psin[pos:pos + 1]
        for h in range(nh):
            want = plain_impl.rope_apply(x[t, h * hd:(h + 1) * hd][None], c, s_, style)[0]
            assert torch.allclose(q_dev[t, h * hd:(h + 1) * hd].float().cpu(), want, atol=tol * 4)
        pg, off = int(table[slots[b], pos // page]), pos % page
        written[pg, off] = True
        for h in range(nkv):
            k = x[t, (nh + h) * hd:(nh + h + 1) * hd]
            want = plain_impl.rope_apply(k[None], c, s_, style)[0]
            assert torch.allclose(kc_dev[pg, h, off].float().cpu(), want, atol=tol * 4)
            v = qkv[t, (nh + nkv + h) * hd:(nh + nkv + h + 1) * hd]
            assert torch.equal(vc_dev[pg, h, off].cpu(), v)
    # nothing else was touched
    untouched = ~written                                                    # [page, offset]
    assert (kc_dev.float().cpu().permute(0, 2, 1, 3)[untouched] == 77.0).all()
    assert (vc_dev.float().cpu().permute(0, 2, 1, 3)[untouched] == 77.0).all()
    # a layer that only reads another layer's cache rotates q and writes nothing
    q2, k2 = d(qkv.clone()), d(kc)
    ops.rope_cache_write(q2, d(torch.from_numpy(cos)), d(torch.from_numpy(sin)), d(token_pos), d(token_seq),
                         d(torch.tensor(slots, dtype=torch.int32)), d(table), k2, k2, n_heads=nh, n_kv_heads=nkv,
                         head_dim=hd, page_size=page, style={"half": 0, "interleaved": 1}[style], write_kv=False)
    assert torch.equal(q2[:, :nh * hd], q_dev[:, :nh * hd]) and (k2.float() == 77.0).all()


@pytest.mark.parametrize("style", ["half", "interleaved"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, hd, bias", [(3, 1, 6, True), (8, 2, 16, False), (28, 4, 128, True)])
def test_rope_and_cache_write_from_accumulators(style, dtype, nh, nkv, hd, bias):
    """The variant fed from float32 accumulators must give what the plain path gives on
    (accumulator + bias), write q to its own buffer and leave the accumulator zeroed."""
    ops = _ops()
    from rust_inference_b200.parts.rope import rope_tables
    page, n_pages = 64, 5
    cos, sin = rope_tables(hd, 10000.0, 200)
    pcos, psin = plain_impl.rope_table(hd, 10000.0, 200)
    table = torch.tensor([[4, 1, 0], [2, 3, 0]], dtype=torch.int32)
    positions, seqs, slots = [0, 70, 127], [0, 1, 1], [1, 0]
    T, width = 3, (nh + 2 * nkv) * hd
    acc = torch.randn(T, width)
    b = torch.randn(width) if bias else None
    d = lambda t: t.to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    acc_dev = d(acc.clone())
    q_out = torch.full((T, nh * hd), 5.0, device=DEV, dtype=dtype)
    kc = torch.zeros(n_pages, nkv, page, hd, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    ops.rope_cache_write_acc(acc_dev, d(b) if bias else None, q_out, d(torch.from_numpy(cos)),
                             d(torch.from_numpy(sin)), i32(positions), i32(seqs), i32(slots), d(table), kc, vc,
                             n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=page,
                             style={"half": 0, "interleaved": 1}[style], write_kv=True)
    assert (acc_dev == 0).all()                                   # clean for the next projection
    x = acc + (b if bias else 0)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    for t in range(T):
        pos, slot = positions[t], slots[seqs[t]]
        c, s_ = pcos[pos:pos + 1], psin[pos:pos + 1]
        pg, off = int(table[slot, pos // page]), pos % page
        for h in range(nh):
            want = plain_impl.rope_apply(x[t, h * hd:(h + 1) * hd][None], c, s_, style)[0]
            assert torch.allclose(q_out[t, h * hd:(h + 1) * hd].float().cpu(), want, atol=tol * 4, rtol=tol)
        for h in range(nkv):
            want = plain_impl.rope_apply(x[t, (nh + h) * hd:(nh + h + 1) * hd][None], c, s_, style)[0]
            assert torch.allclose(kc[pg, h, off].float().cpu(), want, atol=tol * 4, rtol=tol)
            v = x[t, (nh + nkv + h) * hd:(nh + nkv + h + 1) * hd]
            assert torch.allclose(vc[pg, h, off].float().cpu(), v, atol=tol * 4, rtol=tol)


GEMM_SHAPES = [(1, 7, 5), (3, 100, 33), (17, 264, 128), (64, 391, 192), (130, 77, 1000), (5, 3584, 64), (300, 130, 520)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m, n, k", GEMM_SHAPES)
def test_gemm_simt_all_epilogues(dtype, m, n, k):
    ops = _ops()
    x = (torch.randn(m, k, device=DEV) * 0.5).to(dtype)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(dtype)
    w2 = (torch.randn(n, k, device=DEV) * 0.1).to(dtype)
    bias = torch.randn(n, device=DEV)
    ref = x.double() @ w.double().t()
    ref2 = x.double() @ w2.double().t()
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    scale = ref.abs().max().item()

    out = torch.empty(m, n, device=DEV, dtype=dtype)
    ops.gemm_simt(x, w, out, ops.EPI_STORE, bias=bias)
    assert (out.double() - (ref + bias)).abs().max().item() <= tol * (scale + bias.abs().max().item())
    out32 = torch.empty(m, n, device=DEV)
    ops.gemm_simt(x, w, out32, ops.EPI_STORE_F32)
    assert (out32.double() - ref).abs().max().item() <= 2e-6 * scale + 1e-30
    res = torch.randn(m, n, device=DEV)
    before = res.clone()
    ops.gemm_simt(x, w, res, ops.EPI_RESIDUAL)
    assert (res.double() - (before + ref)).abs().max().item() <= 2e-6 * (scale + 4)
    act = torch.empty(m, n, device=DEV, dtype=dtype)
    ops.gemm_simt(x, w, act, ops.EPI_SILU_MUL, w2=w2)
    want = plain_impl.silu(ref.float()).double() * ref2
    assert (act.double() - want).abs().max().item() <= tol * (want.abs().max().item() + 1e-3) * 2


@pytest.mark.parametrize("m", [1, 8, 33, 64, 100, 130, 300, 700])
@pytest.mark.parametrize("n, k", [(128, 64), (391, 192), (200, 136), (640, 1032), (3584, 3584)])
def test_gemm_tcgen05_all_epilogues(m, n, k):
    """bf16 operands on the tensor cores: every token tile (16..256), ragged features and K."""
    ops = _ops()
    from rust_inference_b200.kernels import linear, tcgen05
    x = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    w = linear.Weight((torch.randn(n, k, device=DEV) * 0.1).bfloat16())
    w2 = linear.Weight((torch.randn(n, k, device=DEV) * 0.1).bfloat16())
    bias = torch.randn(n, device=DEV)
    assert tcgen05.supports(x, w)
    ref = x.double() @ w.t.double().t()
    ref2 = x.double() @ w2.t.double().t()
    scale = ref.abs().max().item()
    out32 = torch.full((m, n), 9.0, device=DEV)
    tcgen05.gemm(x, w, out32, ops.EPI_STORE_F32)
    assert (out32.double() - ref).abs().max().item() <= 1e-5 * scale           # float32 accumulation
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    tcgen05.gemm(x, w, out, ops.EPI_STORE, bias=bias)
    assert (out.double() - (ref + bias)).abs().max().item() <= 8e-3 * (scale + bias.abs().max().item())
    for split in (1, 3):
        res = torch.randn(m, n, device=DEV)
        before = res.clone()
        tcgen05.gemm(x, w, res, ops.EPI_RESIDUAL, split_k=split)
        assert (res.double() - (before + ref)).abs().max().item() <= 1e-5 * (scale + 4)
    act = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    tcgen05.gemm(x, w, act, ops.EPI_SILU_MUL, w2=w2)
    want = plain_impl.silu(ref.float()).double() * ref2
    assert (act.double() - want).abs().max().item() <= 8e-3 * (want.abs().max().item() + 1e-3)
    torch.cuda.synchronize()
    tcgen05.check_status()


@pytest.mark.parametrize("m, n, k", [(2048, 3584, 256), (1111, 1000, 72), (257, 19 * 128, 64)])
def test_gemm_tcgen05_token_tile_follows_the_grid(m, n, k):
    """Long steps run the token tile of 128..256 rows, and the residual epilogue the K split, that
    leave the shortest run in the persistent grid; however a product is cut, it is the same product."""
    ops = _ops()
    from rust_inference_b200.kernels import linear, tcgen05
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    kb = -(-k // 64)
    for mode in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL):
        tn, split = tcgen05.plan(m, n, k, mode)
        assert 128 <= tn <= 256 and tn % 16 == 0 and 1 <= split <= max(1, kb // 4)
        assert split == 1 or mode == ops.EPI_RESIDUAL
        splits = range(1, max(1, min(10, kb // 4)) + 1) if mode == ops.EPI_RESIDUAL else (1,)
        cost = lambda t, s: -(-(-(-m // t) * -(-n // 128) * s) // sms) * (-(-kb // s) + 12)
        assert cost(tn, split) == min(cost(t, s) for t in range(128, 257, 16) for s in splits)
    x = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    w = linear.Weight((torch.randn(n, k, device=DEV) * 0.1).bfloat16())
    ref = x.double() @ w.t.double().t()
    out32 = torch.full((m, n), 9.0, device=DEV)
    tcgen05.gemm(x, w, out32, ops.EPI_STORE_F32)
    assert (out32.double() - ref).abs().max().item() <= 1e-5 * ref.abs().max().item()
    res = torch.randn(m, n, device=DEV)
    before = res.clone()
    tcgen05.gemm(x, w, res, ops.EPI_RESIDUAL)
    assert (res.double() - (before + ref)).abs().max().item() <= 1e-5 * (ref.abs().max().item() + 4)
    torch.cuda.synchronize()
    tcgen05.check_status()


@pytest.mark.parametrize("m, n, k", [(512, 512, 256), (300, 1000, 520), (1111, 264, 72), (256, 3000, 64), (40, 384, 128),
                                     (2048, 1184, 1096)])
def test_gemm_tcgen05_on_pairs_of_sms(m, n, k):
    """The same products with two CTAs sharing each MMA (tcgen05 cta_group::2: 256 tokens x 256 weight rows per
    pair, each CTA loading half of both operands), forced on whatever the shape; ragged tokens, features and K."""
    ops = _ops()
    from rust_inference_b200.kernels import linear, tcgen05
    tcgen05.set_pairs(1, always=True)
    try:
        assert tcgen05.plan(m, n, k, ops.EPI_STORE) == (128, 1)
        x = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
        w = linear.Weight((torch.randn(n, k, device=DEV) * 0.1).bfloat16())
        w2 = linear.Weight((torch.randn(n, k, device=DEV) * 0.1).bfloat16())
        bias = torch.randn(n, device=DEV)
        ref = x.double() @ w.t.double().t()
        ref2 = x.double() @ w2.t.double().t()
        scale = ref.abs().max().item()
        out32 = torch.full((m, n), 9.0, device=DEV)
        tcgen05.gemm(x, w, out32, ops.EPI_STORE_F32)
        assert (out32.double() - ref).abs().max().item() <= 1e-5 * scale
        out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
        tcgen05.gemm(x, w, out, ops.EPI_STORE, bias=bias)
        assert (out.double() - (ref + bias)).abs().max().item() <= 8e-3 * (scale + bias.abs().max().item())
        act = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
        tcgen05.gemm(x, w, act, ops.EPI_SILU_MUL, w2=w2)
        want = plain_impl.silu(ref.float()).double() * ref2
        assert (act.double() - want).abs().max().item() <= 8e-3 * (want.abs().max().item() + 1e-3)
        # the adding epilogue stays with the single-CTA kernel, which can split K
        res = torch.randn(m, n, device=DEV)
        before = res.clone()
        tcgen05.gemm(x, w, res, ops.EPI_RESIDUAL)
        assert (res.double() - (before + ref)).abs().max().item() <= 1e-5 * (scale + 4)
        torch.cuda.synchronize()
        tcgen05.check_status()
    finally:
        tcgen05.set_pairs()
    # by default only long steps whose tiles fill the pairs' rounds go there
    assert tcgen05.plan(8, 3584, 3584, ops.EPI_STORE)[0] == 16
    assert tcgen05.plan(2048, 18944, 3584, ops.EPI_SILU_MUL) == (128, 1)


def test_gemm_tcgen05_refuses_what_it_cannot_do():
    from rust_inference_b200.kernels import linear, ops, tcgen05
    x = torch.zeros(4, 100, device=DEV, dtype=torch.bfloat16)
    w = linear.Weight(torch.zeros(8, 100, device=DEV, dtype=torch.bfloat16))
    assert not tcgen05.supports(x, w)                     # rows of 200 bytes: not a multiple of 16
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        tcgen05.gemm(x, w, torch.zeros(4, 8, device=DEV), ops.EPI_STORE_F32)
    # the dispatcher takes the FFMA kernel for such a shape instead
    out = torch.empty(4, 8, device=DEV)
    linear.logits(x, w, out, None)
    assert (out == 0).all()
    with pytest.raises(ops.KernelError, match="CUDA"):
        ops.rmsnorm(torch.zeros(2, 4), torch.ones(4), 1e-5, torch.zeros(2, 4))


def _attention_case(nh, nkv, hd, news, starts, dtype, window=0, sharp=None, seed=0):
    """Random q, K, V in a scrambled paged cache; returns the kernel inputs and the plain result."""
    g = torch.Generator().manual_seed(seed)
    page = 64
    B = len(news)
    total = [s + n for s, n in zip(starts, news)]
    max_pages = max(-(-t // page) for t in total) + 1
    n_pages = sum(-(-t // page) for t in total) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    slots = list(range(B - 1, -1, -1))
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    kc = torch.randn(n_pages, nkv, page, hd, generator=g).to(dtype)         # unused places hold noise
    vc = torch.randn(n_pages, nkv, page, hd, generator=g).to(dtype)
    Ks, Vs, pi = [], [], 0
    for b in range(B):
        K = torch.randn(total[b], nkv, hd, generator=g).to(dtype)
        V = torch.randn(total[b], nkv, hd, generator=g).to(dtype)
        if sharp is not None:
            K[sharp % total[b]] *= 6.0                                       # one key stands out
        Ks.append(K)
        Vs.append(V)
        for pg in range(-(-total[b] // page)):
            p = perm[pi]
            pi += 1
            table[slots[b], pg] = p
            n = min(page, total[b] - pg * page)
            kc[p, :, :n] = K[pg * page:pg * page + n].transpose(0, 1)
            vc[p, :, :n] = V[pg * page:pg * page + n].transpose(0, 1)
    T = sum(news)
    q = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    scale = 1.0 / math.sqrt(hd)
    ref = torch.zeros(T, nh * hd)
    rep = nh // nkv
    for b in range(B):
        for i in range(news[b]):
            t, pos = cu[b] + i, starts[b] + i
            lo = max(0, pos - window + 1) if window > 0 else 0
            for h in range(nh):
                k = Ks[b][lo:pos + 1, h // rep].float()
                v = Vs[b][lo:pos + 1, h // rep].float()
                s = (k @ q[t, h * hd:(h + 1) * hd].float()) * scale
                ref[t, h * hd:(h + 1) * hd] = plain_impl.softmax_rows(s[None])[0] @ v
    d = lambda t: t.to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    pos = [starts[b] + i for b in range(B) for i in range(news[b])]
    seq = [b for b in range(B) for _ in range(news[b])]
    return dict(q=d(q), kc=d(kc), vc=d(vc), table=d(table), slot=i32(slots), start=i32(starts), length=i32(total),
                cu=i32(cu), pos=i32(pos), seq=i32(seq), ref=ref, scale=scale, T=T, B=B)


ATTN_CASES = [
    (2, 1, 128, [300], [0], 0),
    (4, 2, 64, [129, 128, 1], [0, 70, 5], 0),
    # heads, kv heads, head_dim, new tokens per sequence, cached before, window
    (4, 2, 64, [5], [0], 0),
    (28, 4, 128, [130, 1, 77], [0, 0, 0], 0),
    (14, 2, 128, [1, 1, 1, 1], [1000, 64, 127, 128], 0),
    (8, 8, 64, [1, 1, 1], [0, 63, 200], 0),
    (6, 3, 64, [33, 2], [100, 700], 0),
    (16, 1, 64, [1], [999], 0),
    (4, 2, 128, [70, 200], [30, 0], 50),
    (4, 1, 64, [1, 1], [300, 5], 100),
    (5, 5, 16, [40, 1], [0, 90], 0),          # head sizes the tensor-core kernels refuse
    (6, 2, 48, [1, 1], [10, 300], 0),
    (3, 1, 80, [20], [50], 30),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, hd, news, starts, window", ATTN_CASES)
def test_attention_kernels(dtype, nh, nkv, hd, news, starts, window):
    ops = _ops()
    c = _attention_case(nh, nkv, hd, news, starts, dtype, window=window)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    out = torch.zeros(c["T"], nh * hd, device=DEV, dtype=dtype)
    ops.attention_generic(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["pos"], c["seq"], c["slot"], out,
                          n_tokens=c["T"], n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=64,
                          scale=c["scale"], window=window)
    assert (out.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item()
    if dtype != torch.bfloat16:
        return
    decode = all(n == 1 for n in news)
    if ops.attention_mma_supports(hd, 64, nh, nkv, False):
        out = torch.zeros_like(out)
        ops.attention_prefill(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["slot"], c["start"], c["cu"],
                              out, n_seqs=c["B"], max_new=max(news), n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                              page_size=64, scale=c["scale"], window=window)
        assert (out.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item()
        from rust_inference_b200.kernels import attention_tc, tcgen05
        assert attention_tc.supports(hd, 64, nh, nkv, c["q"].shape[1], nh * hd)
        out = torch.zeros_like(out)
        attention_tc.prefill(c["q"], c["kc"], c["vc"], c["table"], c["slot"], c["start"], c["cu"], out,
                             n_seqs=c["B"], max_new=max(news), n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                             page_size=64, scale=c["scale"], window=window)
        torch.cuda.synchronize()
        tcgen05.check_status()
        assert (out.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item()
    else:
        assert hd not in (64, 128)
    if decode and ops.attention_mma_supports(hd, 64, nh, nkv, True):
        for splits in (1, 2, 7, 32):
            out = torch.zeros_like(out)
            po = torch.full((c["B"] * nh * splits * hd,), float("nan"), device=DEV)
            pml = torch.full((c["B"] * nh * splits * 2,), float("nan"), device=DEV)
            ops.attention_decode(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["slot"], c["length"],
                                 c["cu"], out, n_seqs=c["B"], n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=64,
                                 scale=c["scale"], window=window, n_splits=splits, part_o=po, part_ml=pml)
            assert (out.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item(), splits
            from rust_inference_b200.kernels import attention_tc, tcgen05
            out2 = torch.zeros_like(out)
            attention_tc.decode(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["slot"], c["length"], c["cu"],
                                out2, n_seqs=c["B"], n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=64,
                                scale=c["scale"], window=window, n_splits=splits, part_o=po, part_ml=pml)
            torch.cuda.synchronize()
            tcgen05.check_status()
            assert (out2.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item(), splits


DECODE_CASES = [
    # heads, kv heads, head_dim, cached before the new token (one per sequence), window
    (14, 2, 128, [1000, 64, 127, 128], 0),
    (8, 8, 64, [0, 63, 200], 0),
    (16, 1, 64, [999], 0),
    (4, 1, 64, [300, 5], 100),
    (28, 4, 128, [1, 0, 511, 700, 64, 65, 1300, 2047], 0),
]


@pytest.mark.parametrize("nh, nkv, hd, starts, window", DECODE_CASES)
def test_decode_attention_as_a_cluster(nh, nkv, hd, starts, window):
    """The runs of a (sequence, kv head) as one thread-block cluster that merges its own partial results."""
    ops = _ops()
    from rust_inference_b200.kernels import attention_tc, tcgen05
    kernel = attention_tc.decode_cluster
    c = _attention_case(nh, nkv, hd, [1] * len(starts), starts, torch.bfloat16, window=window)
    for splits in (2, 3, 5, 8):
        out = torch.zeros(c["T"], nh * hd, device=DEV, dtype=torch.bfloat16)
        kernel(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["slot"], c["length"],
               c["cu"], out, n_seqs=c["B"], n_heads=nh, n_kv_heads=nkv, head_dim=hd,
               page_size=64, scale=c["scale"], window=window, n_splits=splits)
        torch.cuda.synchronize()
        tcgen05.check_status()
        assert (out.float().cpu() - c["ref"]).abs().max().item() <= 2e-2 * c["ref"].abs().max().item(), splits
    with pytest.raises(ops.KernelError, match="2 to 8 splits"):
        kernel(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["slot"], c["length"],
               c["cu"], out, n_seqs=c["B"], n_heads=nh, n_kv_heads=nkv, head_dim=hd,
               page_size=64, scale=c["scale"], window=window, n_splits=9)
    assert attention_tc.decode_cluster_capacity(hd, 8) >= 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key(dtype):
    """One key among hundreds is scaled up so that its score stands out: the result must be
    (nearly) that key's value, wherever the key lies (first page, a page boundary, the last key)."""
    ops = _ops()
    nh, nkv, hd = 4, 2, 64
    for far in (0, 63, 64, 500, 898):
        c = _attention_case(nh, nkv, hd, [1, 3], [898, 897], dtype, sharp=far, seed=far)
        out = torch.zeros(c["T"], nh * hd, device=DEV, dtype=dtype)
        ops.attention_generic(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["pos"], c["seq"], c["slot"],
                              out, n_tokens=c["T"], n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=64,
                              scale=c["scale"])
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (out.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item()
        if dtype == torch.bfloat16:
            out2 = torch.zeros_like(out)
            ops.attention_prefill(c["q"], c["q"].shape[1], c["kc"], c["vc"], c["table"], c["slot"], c["start"],
                                  c["cu"], out2, n_seqs=2, max_new=3, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                                  page_size=64, scale=c["scale"], window=0)
            assert (out2.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item()
            from rust_inference_b200.kernels import attention_tc
            out3 = torch.zeros_like(out)
            attention_tc.prefill(c["q"], c["kc"], c["vc"], c["table"], c["slot"], c["start"], c["cu"], out3, n_seqs=2,
                                 max_new=3, n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_size=64, scale=c["scale"])
            assert (out3.float().cpu() - c["ref"]).abs().max().item() <= tol * c["ref"].abs().max().item()


@pytest.fixture(params=["a block per row", "a cluster per row"])
def sampling_kernel(request):
    """Every sampling test runs twice: with the kernel that gives a row to one thread block, and with the one
    that gives it to a cluster of eight wherever the options allow it (whatever the size of the vocabulary)."""
    ops = _ops()
    ops.sample_cluster_min_vocab(0 if request.param == "a block per row" else 1)
    ops.sample_cluster_any_rows(True)
    yield request.param
    ops.sample_cluster_min_vocab(32768)
    ops.sample_cluster_any_rows(False)


def _sample(logits, **kw):
    ops = _ops()
    rows = logits.shape[0]
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    kw.setdefault("row_stream", i32(list(range(rows))))
    kw.setdefault("row_counter", i32([0] * rows))
    ops.sample(logits.clone().to(DEV), out, **kw)
    return out.cpu().tolist()


def test_sampling_greedy_first_maximum(sampling_kernel):
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(6, 152064, generator=g)
    logits[1, 777] = logits[1, 151000] = 50.0                 # a tie: the first wins (math.rs:328-339)
    logits[2, 0] = 60.0
    logits[3, 152063] = 60.0
    logits[4] = 1.0                                            # all equal
    got = _sample(logits, temperature=0.0)
    assert got == [plain_impl.argmax_first(logits[i]) for i in range(6)]
    assert got[1] == 777 and got[2] == 0 and got[3] == 152063 and got[4] == 0
    small = torch.tensor([[0.1, 0.7, 0.7], [-1.0, -3.0, -0.5]])
    assert _sample(small, temperature=0.0) == [1, 2]


@pytest.mark.parametrize("vocab", [5, 384, 1000, 152064])
def test_sampling_temperature_matches_the_cdf(vocab, sampling_kernel):
    """The drawn token must be the one whose CDF interval holds u, up to rounding at the edges."""
    g = torch.Generator().manual_seed(vocab)
    rows, T, seed = 64, 0.7, 4
    logits = torch.randn(rows, vocab, generator=g) * 3
    counters = [(3 * r) % 11 for r in range(rows)]
    got = _sample(logits, temperature=T, seed=seed,
                  row_counter=torch.tensor(counters, dtype=torch.int32, device=DEV))
    for r in range(rows):
        u = rng.uniform(seed, r, counters[r])
        cdf = torch.cumsum(torch.softmax(logits[r].double() / T, dim=0), dim=0)
        lo = cdf[got[r] - 1].item() if got[r] > 0 else 0.0
        assert lo - 1e-5 <= u <= cdf[got[r]].item() + 1e-5, (r, got[r], u)
        if vocab <= 1000:
            probs = plain_impl.softmax_rows((logits[r] / T)[None])[0]
            assert got[r] == plain_impl.draw(probs, u) or abs(cdf[got[r]].item() - u) < 1e-5 or abs(lo - u) < 1e-5


def test_sampling_frequencies_follow_the_distribution(sampling_kernel):
    probs = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625])
    n = 4000
    logits = probs.log()[None].repeat(n, 1)
    got = _sample(logits, temperature=1.0, seed=99)
    freq = torch.bincount(torch.tensor(got), minlength=5).float() / n
    assert (freq - probs).abs().max().item() < 0.03


def test_sampling_top_k_top_p_and_penalty_follow_the_reference(sampling_kernel):
    g = torch.Generator().manual_seed(1)
    vocab, rows, seed = 500, 48, 7
    logits = torch.randn(rows, vocab, generator=g) * 2
    logits[:, 10] = logits[:, 20]                               # ties inside the distribution
    recent = torch.randint(0, vocab, (rows, 8), generator=g).int()
    counts = torch.tensor([r % 9 for r in range(rows)], dtype=torch.int32)
    for kw in (dict(top_k=5), dict(top_p=0.6), dict(top_k=40, top_p=0.95), dict(top_k=1),
               dict(top_k=40, top_p=0.95, penalty=1.1), dict(penalty=1.5), dict(top_p=0.999)):
        use_recent = "penalty" in kw
        got = _sample(logits, temperature=0.8, seed=seed, **kw,
                      **({"recent": recent.to(DEV), "recent_count": counts.to(DEV)} if use_recent else {}))
        for r in range(rows):
            u = rng.uniform(seed, r, 0)
            hist = recent[r, :counts[r]].tolist() if use_recent else []
            l = plain_impl.repetition_penalty(logits[r], hist, kw.get("penalty", 1.0), 64) if hist else logits[r]
            p = plain_impl.softmax_rows((l.double() / 0.8)[None])[0]
            p = plain_impl.top_k_filter(p, kw.get("top_k", 0))
            p = plain_impl.top_p_filter(p, kw.get("top_p", 1.0))
            assert p[got[r]] > 0, (kw, r, "a filtered token was drawn")
            cdf = torch.cumsum(p, dim=0)
            lo = cdf[got[r] - 1].item() if got[r] > 0 else 0.0
            assert lo - 2e-5 <= u <= cdf[got[r]].item() + 2e-5, (kw, r, got[r], u)
    # greedy after a penalty (sampler.rs:76-83): the penalised maximum loses
    l = torch.tensor([[1.0, 5.0, 4.9, -2.0]])
    assert _sample(l, temperature=0.0) == [1]
    assert _sample(l, temperature=0.0, penalty=1.1, recent=torch.tensor([[1]], dtype=torch.int32, device=DEV),
                   recent_count=torch.tensor([1], dtype=torch.int32, device=DEV)) == [2]


def test_sampling_penalises_an_id_as_often_as_it_occurs(sampling_kernel):
    """The recent ids may name a token several times, and the newest one (on the device) may repeat one of
    them: each occurrence applies the penalty again (sampler.rs:109-127).  Greedy leaves the penalised logits
    in the buffer, which is compared entry by entry."""
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    for vocab in (50, 40000):
        rows = 5
        logits = torch.randn(rows, vocab, generator=g) * 4
        recent = torch.randint(0, vocab, (rows, 64), generator=g).int()
        recent[:, 10:20] = recent[:, 0:1]                      # the first id another ten times
        recent[:, 30] = recent[:, 31] = vocab - 1
        counts = torch.tensor([64, 33, 0, 12, 64], dtype=torch.int32)
        newest = recent[:, 0].clone()
        newest[3] = 7
        buf = logits.clone().to(DEV)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        ops.sample(buf, out, temperature=0.0, penalty=1.3, recent=recent.to(DEV), recent_count=counts.to(DEV),
                   newest=newest.to(DEV))
        for r in range(rows):
            hist = recent[r, :counts[r]].tolist() + [int(newest[r])]
            want = plain_impl.repetition_penalty(logits[r], hist, 1.3, 10 ** 6)
            assert torch.allclose(buf[r].cpu(), want, rtol=1e-6, atol=0), (vocab, r)
            assert out[r].item() == plain_impl.argmax_first(want)


@pytest.mark.parametrize("vocab, kw", [
    (152064, dict(top_k=40, top_p=0.95)), (152064, dict(top_k=1000)), (152064, dict(top_k=1024, top_p=0.5)),
    (4099, dict(top_k=7)), (5, dict(top_k=3, top_p=0.9)), (37, dict(top_k=36)), (152064, dict(top_k=256)),
    (40001, dict(top_k=200, top_p=0.8)), (33000, dict(top_k=2)),
])
def test_sampling_top_k_over_a_candidate_list(vocab, kw, sampling_kernel):
    """With top-k the kernel keeps a short list of candidates instead of walking the vocabulary for every
    threshold: the drawn token must lie where the plain filters put the uniform number."""
    g = torch.Generator().manual_seed(vocab)
    rows, seed = 6, 11
    logits = torch.randn(rows, vocab, generator=g) * 3
    logits[:, 1] = logits[:, 3]
    got = _sample(logits, temperature=0.7, seed=seed, **kw)
    for r in range(rows):
        u = rng.uniform(seed, r, 0)
        p = plain_impl.softmax_rows((logits[r].double() / 0.7)[None])[0]
        p = plain_impl.top_k_filter(p, kw.get("top_k", 0))
        p = plain_impl.top_p_filter(p, kw.get("top_p", 1.0))
        assert p[got[r]] > 0, (kw, r, "a filtered token was drawn")
        cdf = torch.cumsum(p, dim=0)
        lo = cdf[got[r] - 1].item() if got[r] > 0 else 0.0
        assert lo - 2e-5 <= u <= cdf[got[r]].item() + 2e-5, (kw, r, got[r], u)


def test_sampling_top_k_with_more_ties_than_the_list_holds(sampling_kernel):
    """Rows in which thousands of ids tie with the k-th largest: every one of them is kept (sampler.rs:130-160
    keeps ties), the candidate list cannot hold them, and the kernel takes the long way."""
    vocab, rows, seed = 20000, 4, 3
    logits = torch.zeros(rows, vocab)
    logits[:, ::2] = 1.0                                             # ten thousand ids share the maximum
    logits[2, 77] = 3.0
    got = _sample(logits, temperature=1.0, seed=seed, top_k=50)
    for r in range(rows):
        u = rng.uniform(seed, r, 0)
        p = plain_impl.softmax_rows(logits[r].double()[None])[0]
        p = plain_impl.top_k_filter(p, 50)
        assert (p > 0).sum() >= 10000 and p[got[r]] > 0
        cdf = torch.cumsum(p, dim=0)
        lo = cdf[got[r] - 1].item() if got[r] > 0 else 0.0
        assert lo - 2e-5 <= u <= cdf[got[r]].item() + 2e-5, (r, got[r], u)


# ----------------------------------------------------------------------------------------
# load-time kernels and the step's own bookkeeping kernel
# ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 255, 256, 100_003])
def test_cast_between_the_two_precisions(n):
    ops = _ops()
    x = torch.randn(n, device=DEV) * 100
    x[0] = 1.00390625                                    # exactly between two bfloat16 values: ties go to even
    down = ops.cast(x, torch.bfloat16)
    assert down.dtype == torch.bfloat16 and torch.equal(down, x.to(torch.bfloat16))
    up = ops.cast(down, torch.float32)
    assert up.dtype == torch.float32 and torch.equal(up, down.float())       # widening is exact


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fill_normal_is_a_function_of_key_and_index(dtype):
    ops = _ops()
    key = 0x1234_5678_9ABC_DEF0
    out = torch.empty(3, 1001, dtype=dtype, device=DEV)
    ops.fill_normal(out, key, mean=1.0, std=0.2)
    flat = out.float().flatten().cpu()
    for i in (0, 1, 2, 1000, 1001, 3002):
        want = 1.0 + 0.2 * rng.normal(key, i)
        tol = 1e-5 if dtype == torch.float32 else 8e-3
        assert abs(float(flat[i]) - want) <= tol, i
    again = torch.empty(3003, dtype=dtype, device=DEV)
    ops.fill_normal(again, key, mean=1.0, std=0.2)
    assert torch.equal(again.flatten(), out.flatten())                   # the shape does not matter
    other = torch.empty(3003, dtype=dtype, device=DEV)
    ops.fill_normal(other, key + 1, mean=1.0, std=0.2)
    assert not torch.equal(other, again)
    big = torch.empty(1 << 20, device=DEV)
    ops.fill_normal(big, 7)
    assert abs(float(big.mean())) < 5e-3 and abs(float(big.std()) - 1.0) < 5e-3
    assert float(big.abs().max()) < 6.0                                  # 24-bit uniforms: |z| <= 5.77


def test_advance_decode_moves_a_step_on():
    ops = _ops()
    n = 300
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    pos, start, length = i32(list(range(n))), i32(list(range(n))), i32([i + 1 for i in range(n)])
    toks = i32([7 * i % 1000 for i in range(n)])
    counter, turn = i32([3] * n), i32([0])
    host = torch.full((4, n), -1, dtype=torch.int32).pin_memory()
    log = torch.full((8, n), -1, dtype=torch.int32, device=DEV)
    for step in range(6):
        toks += 1
        ops.advance_decode(pos, start, length, toks, draw_counter=counter, turn=turn, host_ring=host, log_ring=log)
    torch.cuda.synchronize()
    assert pos.tolist() == [i + 6 for i in range(n)] and start.tolist() == pos.tolist()
    assert length.tolist() == [i + 7 for i in range(n)] and counter.tolist() == [9] * n and turn.item() == 6
    final = toks.cpu()
    assert torch.equal(host[5 % 4], final) and torch.equal(host[4 % 4], final - 1)     # the ring's last two slots
    assert torch.equal(log[5].cpu(), final) and torch.equal(log[0].cpu(), final - 5)
    # without the optional parts only the three arrays move
    ops.advance_decode(pos, start, length, toks)
    assert pos[0].item() == 7 and turn.item() == 6
