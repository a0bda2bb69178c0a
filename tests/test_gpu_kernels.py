"""Each kernel alone against a plain 32-bit (or 64-bit) computation of the same operation, at sizes
other than the engine's: widths and vocabularies that are no power of two, head sizes in steps of
16, odd head counts and groups, page edges, a far key among hundreds, a window's edge."""
import math

import numpy as np
import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def K():
    from geneinfer_b200.ops import kernels
    return kernels


def dt(name):
    return torch.float32 if name == "float32" else torch.bfloat16


def close(got, want, dtype, what, f32_tol=2e-6, bf16_tol=1e-2):
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all(), f"{what}: not finite"
    tol = f32_tol if dtype == "float32" else bf16_tol
    err = float((got - want).abs().max() / max(1.0, float(want.abs().max())))
    assert err < tol, f"{what}: error {err:.3e} >= {tol:.1e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,V", [(1, 48, 37), (19, 200, 1000), (130, 2048 + 16, 511)])
def test_embed(dtype, T, D, V):
    g = torch.Generator().manual_seed(1)
    table = torch.randn(V, D, generator=g).to(dt(dtype)).to(DEV)
    tokens = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.full((T, D), float("nan"), device=DEV)
    K().embed(table, tokens, out, 1.0)
    assert torch.equal(out.cpu(), table.float().cpu()[tokens.cpu().long()])


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,eps", [(1, 16, 1e-5), (7, 96, 1e-6), (33, 1000, 0.05), (5, 4096 + 48, 1e-5)])
def test_rmsnorm(out_dtype, T, D, eps):
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(T, D, generator=g) * 3).to(DEV)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(DEV)
    out = torch.full((T, D), float("nan"), dtype=dt(out_dtype), device=DEV)
    K().rmsnorm(x, w, out, eps)
    want = pm.plain_rmsnorm(x.cpu(), w.cpu(), eps)
    close(out, want, out_dtype, "rmsnorm")
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    out2 = torch.full((3, D), float("nan"), dtype=dt(out_dtype), device=DEV)
    K().rmsnorm(x, w, out2, eps, rows)
    assert torch.equal(out2.cpu(), out.cpu()[rows.cpu().long()]), "gathered rows differ from the same rows in place"


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,I", [(1, 16), (9, 160), (64, 1000), (5, 30), (3, 8192 + 2)])
def test_swiglu(out_dtype, T, I):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(T, 2 * I, generator=g) * 4).to(DEV)
    out = torch.full((T, I), float("nan"), dtype=dt(out_dtype), device=DEV)
    K().swiglu(gu, out)
    close(out, pm.plain_swiglu(gu.cpu()[:, :I], gu.cpu()[:, I:]), out_dtype, "swiglu")


@pytest.mark.parametrize("a_dtype,w_dtype,c_dtype", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "float32"),
                                                     ("bfloat16", "bfloat16", "bfloat16"), ("float32", "bfloat16", "float32")])
@pytest.mark.parametrize("M,N,K_", [(1, 1, 1), (1, 384, 96), (7, 100, 33), (65, 129, 257), (200, 64, 1000)])
def test_gemm_simt(a_dtype, w_dtype, c_dtype, M, N, K_):
    g = torch.Generator().manual_seed(4)
    a = torch.randn(M, K_, generator=g).to(dt(a_dtype)).to(DEV)
    w = torch.randn(N, K_, generator=g).to(dt(w_dtype)).to(DEV)
    want = a.float().cpu().double() @ w.float().cpu().double().T
    out = torch.full((M, N), float("nan"), dtype=dt(c_dtype), device=DEV)
    K().gemm_simt(a, w, out)
    close(out, want, c_dtype, "gemm", f32_tol=1e-5)
    if c_dtype == "float32":
        base = torch.randn(M, N, generator=g).to(DEV)
        acc = base.clone()
        K().gemm_simt(a, w, acc, accumulate=True)
        close(acc, want + base.cpu().double(), "float32", "gemm accumulate", f32_tol=1e-5)
        if M > 1:   # a row's result does not depend on the rows around it
            one = torch.empty((1, N), device=DEV)
            K().gemm_simt(a[M - 1:M].contiguous(), w, one)
            assert torch.equal(one[0], out[M - 1]), "a row alone differs from the row in the batch"


def _paged(dtype, n_pages, Hkv, ps, hd):
    kc = torch.full((n_pages, Hkv, ps, hd), float("nan"), dtype=dt(dtype), device=DEV)
    return kc, kc.clone()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hkv,hd,ps,interleaved,rot", [(4, 2, 16, 16, False, 16), (3, 1, 32, 8, False, 32),
                                                          (6, 3, 48, 4, True, 48), (2, 2, 64, 16, False, 32)])
def test_rope_store(dtype, H, Hkv, hd, ps, interleaved, rot):
    g = torch.Generator().manual_seed(5)
    lens = [5, 1, 2 * ps + 3]                         # three requests; rows: a portion, one token, a portion over a page edge
    first = [ps - 2, 3 * ps - 1, 0]                   # the first portion crosses a page edge, the single token ends a page
    T = sum(lens)
    qkv = torch.randn(T, (H + 2 * Hkv) * hd, generator=g).to(DEV)
    max_pos = 4 * ps
    freq = 1.0 / (10000.0 ** (np.arange(rot // 2, dtype=np.float64) * 2 / rot))
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * freq[None]
    cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(DEV)
    sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(DEV)
    n_pages = 16
    perm = torch.randperm(n_pages, generator=g).int()
    tables = torch.full((3, 4), -1, dtype=torch.int32)
    k_used = 0
    for r in range(3):
        for i in range((first[r] + lens[r] + ps - 1) // ps):
            tables[r, i] = perm[k_used]
            k_used += 1
    positions = torch.cat([torch.arange(first[r], first[r] + lens[r]) for r in range(3)]).int()
    row_req = torch.cat([torch.full((lens[r],), r) for r in range(3)]).int()
    kc, vc = _paged(dtype, n_pages, Hkv, ps, hd)
    q_out = torch.full((T, H * hd), float("nan"), dtype=dt(dtype), device=DEV)
    K().rope_store(qkv, positions.to(DEV), row_req.to(DEV), tables.to(DEV), cos, sin, interleaved, q_out, kc, vc,
                   H, Hkv, hd, ps)
    x = qkv.cpu().reshape(T, H + 2 * Hkv, hd)

    def rotate(v, p):      # [heads, hd]
        out = v.clone()
        c, s = cos.cpu()[p], sin.cpu()[p]
        half = rot // 2
        if interleaved:
            a, b = v[:, 0:rot:2], v[:, 1:rot:2]
            out[:, 0:rot:2], out[:, 1:rot:2] = a * c - b * s, a * s + b * c
        else:
            a, b = v[:, :half], v[:, half:rot]
            out[:, :half], out[:, half:rot] = a * c - b * s, a * s + b * c
        return out

    written = torch.zeros(n_pages, ps, dtype=torch.bool)
    for t in range(T):
        p, r = int(positions[t]), int(row_req[t])
        close(q_out[t].reshape(H, hd), rotate(x[t, :H], p), dtype, f"q row {t}")
        page, off = int(tables[r, p // ps]), p % ps
        close(kc[page, :, off], rotate(x[t, H:H + Hkv], p), dtype, f"k row {t}")
        close(vc[page, :, off], x[t, H + Hkv:], dtype, f"v row {t}")
        written[page, off] = True
    untouched = ~written
    assert torch.isnan(kc.float().cpu().permute(0, 2, 1, 3)[untouched]).all() and \
        torch.isnan(vc.float().cpu().permute(0, 2, 1, 3)[untouched]).all(), \
        "rows of other positions were written"


def _run_fast_attention(q_all, kc, vc, out, row_req, positions, tables, q_lens, ctx_lens, H, Hkv, hd, ps, scale, window,
                        tcgen05=False, decode_chunks=None):
    """The tensor-core kernels: single tokens through the decode kernel, portions through prefill."""
    kern = K()
    G = H // Hkv
    per_tile = (128 if tcgen05 else kern.attention_prefill_rows(ps, hd)) // G
    decode_rows, work, row = [], [], 0
    for r, n in enumerate(q_lens):
        if n == 1:
            decode_rows.append(row)
        else:
            for t in range(0, n, per_tile):
                work.append([row + t, min(per_tile, n - t), r])
        row += n
    if decode_rows:
        chunk = kern.attention_chunk_keys()
        max_chunks = (max(ctx_lens) + chunk - 1) // chunk + 2
        n_chunks = decode_chunks or (max(ctx_lens[r] for r, n in enumerate(q_lens) if n == 1) + chunk - 1) // chunk
        part_o = torch.full((len(decode_rows) * H * max_chunks * hd,), float("nan"), device=DEV)
        part_ml = torch.full((len(decode_rows) * H * max_chunks * 2,), float("nan"), device=DEV)
        kern.attention_decode(q_all, kc, vc, out, torch.tensor(decode_rows, dtype=torch.int32, device=DEV), row_req,
                              positions, tables, H, Hkv, hd, ps, scale, window, part_o, part_ml, max_chunks, n_chunks)
    if work:
        fn = kern.attention_prefill_tc if tcgen05 else kern.attention_prefill
        fn(q_all, kc, vc, out, torch.tensor(work, dtype=torch.int32, device=DEV), positions, tables, H, Hkv, hd, ps, scale, window)


def _attention_case(dtype, H, Hkv, hd, ps, ctx_lens, q_lens, window, seed, spike=None, fast=False, tcgen05=False,
                    decode_chunks=None):
    """Requests with ``ctx_lens`` cached positions of which the last ``q_lens`` are this step's
    queries. Pages are scattered and unused pages hold NaN. ``spike`` = (request, key position):
    that key is made to match every query of the request strongly."""
    g = torch.Generator().manual_seed(seed)
    R = len(ctx_lens)
    n_pages = sum((c + ps - 1) // ps for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=g).int()
    stride = max((c + ps - 1) // ps for c in ctx_lens)
    tables = torch.full((R, stride), -1, dtype=torch.int32)
    kc, vc = _paged(dtype, n_pages, Hkv, ps, hd)
    ks, vs, qs, positions, row_req = [], [], [], [], []
    used = 0
    for r in range(R):
        k = torch.randn(ctx_lens[r], Hkv, hd, generator=g)
        v = torch.randn(ctx_lens[r], Hkv, hd, generator=g)
        q = torch.randn(ctx_lens[r], H, hd, generator=g)        # a query for every position; only the last q_lens run
        if spike and spike[0] == r:
            direction = torch.randn(hd, generator=g)
            direction /= direction.norm()
            k[spike[1]] = 12.0 * direction
            q[:] = q * 0.3 + 12.0 * direction
            v[spike[1]] = 5.0
        k, v, q = (t.to(dt(dtype)).float() for t in (k, v, q))
        for i in range((ctx_lens[r] + ps - 1) // ps):
            page = int(perm[used]); used += 1
            tables[r, i] = page
            n = min(ps, ctx_lens[r] - i * ps)
            kc[page, :, :n] = k[i * ps:i * ps + n].transpose(0, 1).to(dt(dtype)).to(DEV)
            vc[page, :, :n] = v[i * ps:i * ps + n].transpose(0, 1).to(dt(dtype)).to(DEV)
        ks.append(k); vs.append(v)
        lo = ctx_lens[r] - q_lens[r]
        qs.append(q[lo:])
        positions += list(range(lo, ctx_lens[r]))
        row_req += [r] * q_lens[r]
    q_all = torch.cat(qs).reshape(-1, H * hd).to(dt(dtype)).to(DEV)
    out = torch.full_like(q_all, float("nan"))
    scale = 1.0 / math.sqrt(hd)
    rr = torch.tensor(row_req, dtype=torch.int32, device=DEV)
    pp = torch.tensor(positions, dtype=torch.int32, device=DEV)
    if fast:
        _run_fast_attention(q_all, kc, vc, out, rr, pp, tables.to(DEV), q_lens, ctx_lens, H, Hkv, hd, ps, scale, window, tcgen05,
                            decode_chunks)
    else:
        K().attention_generic(q_all, kc, vc, out, rr, pp, tables.to(DEV), H, Hkv, hd, ps, scale, window)
    want = []
    for r in range(R):
        full_q = torch.zeros(ctx_lens[r], H, hd)
        full_q[ctx_lens[r] - q_lens[r]:] = qs[r]
        o = pm.plain_attention(full_q, ks[r], vs[r], scale, window)
        want.append(o[ctx_lens[r] - q_lens[r]:])
    return out.reshape(-1, H, hd), torch.cat(want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hkv,hd,ps", [(4, 2, 16, 16), (3, 1, 32, 8), (6, 3, 48, 16), (8, 2, 128, 32), (2, 1, 256, 16),
                                          (5, 5, 80, 4)])
def test_attention_mixed_rows(dtype, H, Hkv, hd, ps):
    # a whole prompt, a single decoded token deep in a context, a portion over page edges, position 0 alone
    got, want = _attention_case(dtype, H, Hkv, hd, ps, ctx_lens=[37, 130, 3 * ps + 1, 1], q_lens=[37, 1, ps + 2, 1],
                                window=None, seed=6)
    close(got, want, dtype, "attention", f32_tol=5e-6, bf16_tol=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 15, 16, 17, 255, 256, 511])
def test_attention_far_key_stands_out(dtype, far):
    """One key among 600 dominates the softmax: an engine that drops it, or reads a neighbour
    instead, returns something else entirely."""
    got, want = _attention_case(dtype, 4, 2, 64, 16, ctx_lens=[600], q_lens=[3], window=None, seed=7, spike=(0, far))
    assert float(want.abs().mean()) > 2.0           # the spiked value dominates the output
    close(got, want, dtype, f"far key {far}", f32_tol=5e-6, bf16_tol=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 16, 33])
def test_attention_window_edge(dtype, window):
    """The key just outside the window is the strong one for the last query and just inside for
    the one before: both sides of the edge are checked."""
    ctx = 100
    got, want = _attention_case(dtype, 4, 2, 32, 16, ctx_lens=[ctx], q_lens=[window + 2], window=window, seed=8,
                                spike=(0, ctx - 1 - window))
    close(got, want, dtype, f"window {window}", f32_tol=5e-6, bf16_tol=1e-2)
    assert float(want[-1].abs().mean()) < 2.0 and float(want[-2].abs().mean()) > 2.0


def test_attention_refuses_unsupported_head_size():
    from geneinfer_b200.ops import KernelError
    with pytest.raises(KernelError, match="head size"):
        _attention_case("float32", 2, 1, 24, 16, [4], [4], None, 1)
    with pytest.raises(KernelError, match="head size"):
        _attention_case("float32", 2, 1, 512, 16, [4], [4], None, 1)


@pytest.mark.parametrize("rows,V", [(1, 1), (3, 1000), (5, 128256), (2, 50257)])
def test_argmax(rows, V):
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(rows, V, generator=g)
    if V > 10:
        logits[0, 7] = logits[0, V - 3] = 50.0       # a tie: the lower index wins
    out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    K().argmax(logits.to(DEV), out)
    want = [int(np.argmax(logits[r].numpy())) for r in range(rows)]
    assert out.cpu().tolist() == want


@pytest.mark.parametrize("V", [5, 384, 1000, 50257])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 5, 1.0), (0.7, 0, 0.9), (1.3, 50, 0.5),
                                                     (1.0, 1, 1.0), (1.0, 0, 1e-6), (2.0, 3, 0.99)])
def test_sample_matches_plain_sampler(V, temperature, top_k, top_p):
    g = torch.Generator().manual_seed(10)
    rows = 24
    logits = (torch.randn(rows, V, generator=g) * 2.5)
    logits[3] = torch.round(logits[3])                # many equal probabilities: index order decides
    logits[4] = 0.0                                   # all equal
    us = torch.rand(rows, generator=g)
    us[0], us[1] = 0.0, float(np.float32(1.0) - np.float32(2.0 ** -24))
    out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows * V, device=DEV)
    K().sample(logits.to(DEV), scratch, torch.full((rows,), temperature, device=DEV),
               torch.full((rows,), top_k, dtype=torch.int32, device=DEV), torch.full((rows,), top_p, device=DEV),
               us.to(DEV), out)
    got = out.cpu().tolist()
    sampler = pm.PlainSampler(temperature, top_k, top_p)
    bad = []
    for r in range(rows):
        want = sampler.sample(logits[r].numpy(), float(us[r]))
        if got[r] != want:
            # a draw that falls within rounding of a boundary of the cumulative sum may land on either side
            lo = pm.PlainSampler(temperature, top_k, top_p).sample(logits[r].numpy(), max(0.0, float(us[r]) - 1e-6))
            hi = pm.PlainSampler(temperature, top_k, top_p).sample(logits[r].numpy(), min(0.99999994, float(us[r]) + 1e-6))
            if got[r] not in (lo, hi):
                bad.append((r, got[r], want))
    assert not bad, f"rows (row, got, want): {bad}"


@pytest.mark.parametrize("M,N,K_,plan", [
    (128, 256, 64, (False, 256, 1)), (128, 256, 512, (False, 256, 1)), (300, 520, 200, (False, 256, 1)),
    (129, 100, 96, (False, 128, 1)), (256, 64, 128, (False, 64, 1)),
    (1, 128, 64, (True, 16, 1)), (7, 384, 96, (True, 16, 1)), (16, 128, 1024, (True, 16, 4)), (8, 2048, 2048, (True, 16, 8)),
    (33, 200, 160, (True, 64, 1)), (64, 300, 1536, (True, 64, 3)), (100, 256, 512, (True, 128, 2)), (20, 130, 264, (True, 32, 2)),
    (24, 300, 2048, (True, 32, 7)), (60, 256, 4096, (True, 64, 6)), (128, 200, 1024, (True, 128, 4)),   # partial tiles in the first split's stages
])
@pytest.mark.parametrize("c_dtype", ["float32", "bfloat16"])
def test_gemm_tensor_cores(M, N, K_, plan, c_dtype):
    """The tcgen05 product in both orientations, with and without the split over K, at sizes that
    are no multiple of the tile in any dimension; rows of zeros beyond M, N and K must not leak."""
    g = torch.Generator().manual_seed(11)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).to(DEV)
    want = a.float().cpu().double() @ w.float().cpu().double().T
    guard = torch.full((M + 2, N), -1024.0, dtype=dt(c_dtype), device=DEV)
    out = guard[1:M + 1]
    out.fill_(float("nan"))
    K().gemm_tc(a, w, out, plan=plan)
    assert K().gemm_tc_status(torch.device(DEV)) == 0
    close(out, want, c_dtype, "gemm_tc", f32_tol=2e-6 * max(1, K_ / 64), bf16_tol=1e-2)
    assert float(guard[0].float().min()) == -1024.0 == float(guard[-1].float().max()), "wrote outside the output"
    if c_dtype == "float32":
        base = torch.randn(M, N, generator=g).to(DEV)
        acc = base.clone()
        K().gemm_tc(a, w, acc, accumulate=True, plan=plan)
        close(acc, want + base.cpu().double(), "float32", "gemm_tc accumulate", f32_tol=2e-6 * max(1, K_ / 64))
        again = torch.empty_like(out)
        K().gemm_tc(a, w, again, plan=plan)
        assert torch.equal(again, out), "two runs differ"
    auto = torch.empty((M, N), dtype=dt(c_dtype), device=DEV)
    K().gemm_tc(a, w, auto)                            # the plan the engine would pick
    close(auto, want, c_dtype, "gemm_tc auto plan", f32_tol=2e-6 * max(1, K_ / 64), bf16_tol=1e-2)
    assert K().gemm_tc_status(torch.device(DEV)) == 0
    if plan[0]:
        # few tokens: the same product with the weights read from their tile-by-tile copy (bulk
        # copies, two blocks of K to a stage); zero padding of the copy must not leak either
        tiles = K().tile_weight(w)
        guard2 = torch.full((M + 2, N), -1024.0, dtype=dt(c_dtype), device=DEV)
        tiled = guard2[1:M + 1]
        tiled.fill_(float("nan"))
        K().gemm_tc(a, w, tiled, plan=plan, w_tiles=tiles)
        close(tiled, want, c_dtype, "gemm_tc tiled", f32_tol=2e-6 * max(1, K_ / 64), bf16_tol=1e-2)
        assert float(guard2[0].float().min()) == -1024.0 == float(guard2[-1].float().max()), "wrote outside the output"
        auto2 = torch.empty((M, N), dtype=dt(c_dtype), device=DEV)
        K().gemm_tc(a, w, auto2, w_tiles=tiles)
        close(auto2, want, c_dtype, "gemm_tc tiled auto plan", f32_tol=2e-6 * max(1, K_ / 64), bf16_tol=1e-2)
        if c_dtype == "float32":
            acc2 = base.clone()
            K().gemm_tc(a, w, acc2, accumulate=True, plan=plan, w_tiles=tiles)
            close(acc2, want + base.cpu().double(), "float32", "gemm_tc tiled accumulate", f32_tol=2e-6 * max(1, K_ / 64))
        assert K().gemm_tc_status(torch.device(DEV)) == 0


def test_tile_weight_layout():
    """Element (r, k) of tile (i, j) lies at r * 64 + ((k // 8) ^ (r % 8)) * 8 + k % 8 of the tile."""
    g = torch.Generator().manual_seed(3)
    w = torch.randn(200, 136, generator=g).to(torch.bfloat16).to(DEV)
    wp = torch.zeros(256, 256, dtype=torch.bfloat16)           # rows and columns padded to multiples of 128
    wp[:200, :136] = w.cpu()
    assert K().tile_weight(w).numel() == 256 * 256
    t = K().tile_weight(w).view(2, 4, 128 * 64).cpu()
    for (i, j, r, k) in [(0, 0, 0, 0), (0, 0, 5, 9), (1, 2, 71, 7), (0, 1, 127, 63), (1, 0, 3, 40), (1, 3, 100, 1)]:
        assert t[i, j, r * 64 + (((k // 8) ^ (r % 8)) * 8) + k % 8] == wp[i * 128 + r, j * 64 + k]


def test_gemm_tensor_cores_refuses_what_tma_cannot_address():
    from geneinfer_b200.ops import KernelError
    a = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)       # K = 100 is no multiple of 8
    w = torch.zeros(8, 100, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="multiples of 8"):
        K().gemm_tc(a, w, torch.empty(4, 8, device=DEV))


@pytest.mark.parametrize("H,Hkv,hd,ps", [(4, 2, 16, 16), (3, 1, 32, 8), (8, 2, 64, 16), (32, 8, 64, 16), (8, 2, 128, 32), (5, 5, 64, 4),
                                          (16, 1, 32, 16), (12, 1, 64, 16), (18, 2, 128, 16)])
def test_attention_tensor_cores_mixed_rows(H, Hkv, hd, ps):
    """The mma kernels on a whole prompt, single tokens deep in long contexts (several chunks, a
    chunk edge, a tile edge), a portion over page edges, and position 0 alone."""
    got, want = _attention_case("bfloat16", H, Hkv, hd, ps, ctx_lens=[150, 700, 3 * ps + 1, 1, 256, 257, 64, 65],
                                q_lens=[150, 1, ps + 2, 1, 1, 1, 1, 1], window=None, seed=6, fast=True)
    close(got, want, "bfloat16", "attention (tensor cores)", bf16_tol=1e-2)


@pytest.mark.parametrize("H,Hkv,hd,ps", [(8, 2, 64, 16), (4, 4, 128, 32), (6, 2, 32, 8), (5, 5, 64, 4)])
@pytest.mark.parametrize("decode_chunks", [1, 3])
def test_attention_decode_contexts_of_one_chunk(H, Hkv, hd, ps, decode_chunks):
    """Single tokens whose keys all lie in one chunk are written by the attention kernel itself: with one
    chunk in the launch no merge kernel runs, with more (the engine rounds the longest context up, or
    another request is longer) the merge kernel leaves them alone. Both give the same bits."""
    outs = []
    for chunks in (decode_chunks, 1):
        got, want = _attention_case("bfloat16", H, Hkv, hd, ps, ctx_lens=[100, 256, 1, 37, 255], q_lens=[1, 1, 1, 1, 1],
                                    window=None, seed=21, fast=True, decode_chunks=chunks)
        close(got, want, "bfloat16", "attention of short contexts", bf16_tol=1e-2)
        outs.append(got)
    assert torch.equal(outs[0], outs[1])
    # a window that lies inside one chunk of a long context is final too
    got, want = _attention_case("bfloat16", H, Hkv, hd, ps, ctx_lens=[700, 520, 300], q_lens=[1, 1, 1], window=40, seed=22,
                                fast=True)
    close(got, want, "bfloat16", "attention of a short window", bf16_tol=1e-2)


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 255, 256, 511, 597])
@pytest.mark.parametrize("q_len", [1, 3])
def test_attention_tensor_cores_far_key(far, q_len):
    got, want = _attention_case("bfloat16", 8, 2, 64, 16, ctx_lens=[600], q_lens=[q_len], window=None, seed=7,
                                spike=(0, far), fast=True)
    assert float(want.abs().mean()) > 2.0
    close(got, want, "bfloat16", f"far key {far}", bf16_tol=1e-2)


@pytest.mark.parametrize("window", [1, 5, 16, 33, 300])
def test_attention_tensor_cores_window_edge(window):
    ctx = 700
    for q_len in (window + 2, 1):      # a portion straddling the edge; and a single token whose edge key is just outside
        got, want = _attention_case("bfloat16", 4, 2, 32, 16, ctx_lens=[ctx], q_lens=[q_len], window=window, seed=8,
                                    spike=(0, ctx - 1 - window), fast=True)
        close(got, want, "bfloat16", f"window {window} q_len {q_len}", bf16_tol=1e-2)
        assert float(want[-1].abs().mean()) < 2.0
    got, want = _attention_case("bfloat16", 4, 2, 32, 16, ctx_lens=[ctx], q_lens=[1], window=window, seed=8,
                                spike=(0, ctx - window), fast=True)          # just inside
    close(got, want, "bfloat16", f"window {window} inside", bf16_tol=1e-2)
    assert float(want[-1].abs().mean()) > 2.0


@pytest.mark.parametrize("M,I,K_", [(129, 128, 64), (300, 200, 96), (256, 1000, 512), (2048, 264, 160)])
def test_gemm_swiglu_fused(M, I, K_):
    """The gate/up product with the activation in its epilogue against the plain two-step form."""
    g = torch.Generator().manual_seed(12)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * I, K_, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    guard = torch.full((M + 2, I), -1024.0, dtype=torch.bfloat16, device=DEV)
    out = guard[1:M + 1]
    out.fill_(float("nan"))
    assert K().gemm_swiglu_supported(M, I, K_)
    K().gemm_swiglu(a, w, out)
    assert K().gemm_tc_status(torch.device(DEV)) == 0
    gu = a.float().cpu().double() @ w.float().cpu().double().T
    want = pm.plain_swiglu(gu[:, :I].float(), gu[:, I:].float())
    close(out, want, "bfloat16", "gemm_swiglu", bf16_tol=1e-2)
    assert float(guard[0].float().min()) == -1024.0 == float(guard[-1].float().max()), "wrote outside the output"


@pytest.mark.parametrize("M,N,K_,block_q", [(128, 256, 64, 256), (1000, 1028, 200, 256), (130, 96, 96, 128), (2048, 3072, 2048, 256),
                                            (517, 384, 160, 128)])
def test_gemm_persistent_many_tiles(M, N, K_, block_q):
    """More tiles than SMs, both accumulator buffers in use, store and add epilogues."""
    g = torch.Generator().manual_seed(13)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).to(DEV)
    want = a.float().cpu().double() @ w.float().cpu().double().T
    out = torch.full((M, N), float("nan"), device=DEV)
    K().gemm_tc(a, w, out, plan=(False, block_q, 1))
    close(out, want, "float32", "persistent store", f32_tol=2e-6 * max(1, K_ / 64))
    base = torch.randn(M, N, generator=g).to(DEV)
    acc = base.clone()
    K().gemm_tc(a, w, acc, accumulate=True, plan=(False, block_q, 1))
    close(acc, want + base.cpu().double(), "float32", "persistent add", f32_tol=2e-6 * max(1, K_ / 64))
    assert K().gemm_tc_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("paired", [True, False])
@pytest.mark.parametrize("M,N,K_,splits", [(129, 256, 64, 1), (257, 528, 200, 1), (385, 272, 136, 1), (640, 1296, 328, 1),
                                           (129, 256, 1032, 3), (513, 300, 2056, 4)])
def test_gemm_on_pairs_of_ctas_and_on_single_ones(M, N, K_, splits, paired, monkeypatch):
    """The many-token product on pairs of CTAs (cta_group::2: 256-row tiles of tokens, each CTA fetching half of the
    weights' tile) and on single CTAs: token counts one past a multiple of 128 and of 256 (a pair whose second CTA has
    a single row, or none), widths that are no multiple of the tile, K cut into ranges; store, add and SwiGLU epilogues."""
    monkeypatch.setattr(K(), "PAIRED_PRODUCTS", paired)
    g = torch.Generator().manual_seed(29)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).to(DEV)
    want = a.float().cpu().double() @ w.float().cpu().double().T
    guard = torch.full((M + 2, N), -1024.0, device=DEV)
    out = guard[1:M + 1]
    out.fill_(float("nan"))
    K().gemm_tc(a, w, out, plan=(False, 256, splits))
    close(out, want, "float32", "store", f32_tol=2e-6 * max(1, K_ / 64))
    assert float(guard[0].min()) == -1024.0 == float(guard[-1].max()), "wrote outside the output"
    base = torch.randn(M, N, generator=g).to(DEV)
    acc = base.clone()
    K().gemm_tc(a, w, acc, accumulate=True, plan=(False, 256, splits))
    close(acc, want + base.cpu().double(), "float32", "add", f32_tol=2e-6 * max(1, K_ / 64))
    if splits == 1 and N % 16 == 0:
        I = N // 2
        h = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        K().gemm_swiglu(a, w, h)
        close(h, pm.plain_swiglu(want[:, :I].float(), want[:, I:].float()), "bfloat16", "swiglu", bf16_tol=1e-2)
    assert K().gemm_tc_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("M,N,K_,block_q,splits", [(512, 2048, 2048, 256, 4), (300, 520, 1032, 256, 3), (130, 256, 520, 256, 2),
                                                   (256, 2048, 8192, 256, 8), (517, 384, 1600, 128, 5), (200, 260, 136, 256, 8)])
def test_gemm_persistent_split_over_k(M, N, K_, block_q, splits):
    """Few output tiles: K is cut into ranges that are work items of their own, added up in order by
    a second kernel; a last range that is shorter, more ranges asked for than blocks exist."""
    g = torch.Generator().manual_seed(19)
    a = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K_, generator=g).to(torch.bfloat16).to(DEV)
    want = a.float().cpu().double() @ w.float().cpu().double().T
    guard = torch.full((M + 2, N), -1024.0, device=DEV)
    out = guard[1:M + 1]
    out.fill_(float("nan"))
    K().gemm_tc(a, w, out, plan=(False, block_q, splits))
    close(out, want, "float32", "persistent split store", f32_tol=2e-6 * max(1, K_ / 64))
    assert float(guard[0].min()) == -1024.0 == float(guard[-1].max()), "wrote outside the output"
    base = torch.randn(M, N, generator=g).to(DEV)
    acc = base.clone()
    K().gemm_tc(a, w, acc, accumulate=True, plan=(False, block_q, splits))
    close(acc, want + base.cpu().double(), "float32", "persistent split add", f32_tol=2e-6 * max(1, K_ / 64))
    again = base.clone()
    K().gemm_tc(a, w, again, accumulate=True, plan=(False, block_q, splits))
    assert torch.equal(again, acc), "two runs differ"
    auto = torch.empty(M, N, device=DEV)
    K().gemm_tc(a, w, auto)
    close(auto, want, "float32", "persistent auto plan", f32_tol=2e-6 * max(1, K_ / 64))
    assert K().gemm_tc_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("H,Hkv,hd,ps", [(8, 2, 64, 16), (32, 8, 64, 16), (3, 1, 64, 8), (8, 2, 128, 32), (5, 5, 64, 16), (4, 4, 128, 128)])
def test_attention_tcgen05_prefill(H, Hkv, hd, ps):
    """The tcgen05 prefill kernel: whole prompts of several key tiles, a portion deep in a context
    over page edges, a two-token portion, with single tokens beside them through the decode kernel."""
    assert K().attention_prefill_tc_supported(hd, H, Hkv, ps)
    got, want = _attention_case("bfloat16", H, Hkv, hd, ps, ctx_lens=[300, 700, 3 * ps + 1, 1, 130, 129], q_lens=[300, 45, ps + 2, 1, 2, 129],
                                window=None, seed=16, fast=True, tcgen05=True)
    assert K().gemm_tc_status(torch.device(DEV)) == 0
    close(got, want, "bfloat16", "attention (tcgen05)", bf16_tol=1e-2)


@pytest.mark.parametrize("far", [0, 127, 128, 255, 256, 500, 597])
def test_attention_tcgen05_far_key(far):
    got, want = _attention_case("bfloat16", 8, 2, 64, 16, ctx_lens=[600], q_lens=[40], window=None, seed=7, spike=(0, far),
                                fast=True, tcgen05=True)
    close(got, want, "bfloat16", f"far key {far}", bf16_tol=1e-2)


@pytest.mark.parametrize("window", [1, 5, 33, 130, 300])
def test_attention_tcgen05_window(window):
    ctx = 700
    got, want = _attention_case("bfloat16", 4, 2, 64, 16, ctx_lens=[ctx], q_lens=[window + 2], window=window, seed=8,
                                spike=(0, ctx - 1 - window), fast=True, tcgen05=True)
    close(got, want, "bfloat16", f"window {window}", bf16_tol=1e-2)
    assert float(want[-1].abs().mean()) < 2.0 and float(want[-2].abs().mean()) > 2.0


@pytest.mark.parametrize("T,H,Hkv,hd,ps,D,rotated", [(300, 5, 1, 64, 16, 192, True), (131, 2, 2, 128, 8, 264, True),
                                                     (257, 3, 3, 32, 16, 128, True), (200, 4, 2, 64, 32, 256, False),
                                                     (8, 5, 1, 64, 16, 192, True), (3, 2, 2, 128, 8, 264, True),
                                                     (40, 6, 2, 32, 16, 128, True), (60, 4, 4, 16, 16, 136, True),
                                                     (24, 6, 2, 32, 16, 1024, True), (31, 3, 1, 64, 8, 2048, True),
                                                     (17, 3, 1, 64, 16, 200, False)])
def test_gemm_rope_store_fused(T, H, Hkv, hd, ps, D, rotated, monkeypatch):
    """The [q; k; v] product with rotation and page store in its epilogue against the product followed by
    the rope+store kernel (and that against exact arithmetic): requests whose rows cross page edges,
    pages in a shuffled order, widths and token counts that fill no tile, untouched pages stay NaN."""
    g = torch.Generator().manual_seed(T + hd)
    n_req = 3
    lens = [T // 2, 1, T - T // 2 - 1]
    first = [ps - 2, 3 * ps - 1, 5]
    max_pos = max(f + n for f, n in zip(first, lens)) + 1
    a = (torch.randn(T, D, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn((H + 2 * Hkv) * hd, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).to(DEV)
    cos = sin = None
    if rotated:
        freq = 1.0 / (10000.0 ** (np.arange(hd // 2, dtype=np.float64) * 2 / hd))
        ang = np.arange(max_pos, dtype=np.float64)[:, None] * freq[None]
        cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(DEV)
        sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(DEV)
    pages_per = [(first[r] + lens[r] + ps - 1) // ps for r in range(n_req)]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=g).int()
    tables = torch.full((n_req, max(pages_per)), -1, dtype=torch.int32)
    used = 0
    for r in range(n_req):
        for i in range(pages_per[r]):
            tables[r, i] = perm[used]
            used += 1
    positions = torch.cat([torch.arange(first[r], first[r] + lens[r]) for r in range(n_req)]).int().to(DEV)
    row_req = torch.cat([torch.full((lens[r],), r) for r in range(n_req)]).int().to(DEV)
    tables = tables.to(DEV)
    monkeypatch.setattr(K(), "_ROPE_FEW_TOKENS", 64)      # the few-token form is built for up to 128 tokens; cover its wider tiles too
    assert K().gemm_rope_store_supported(T, D, H, Hkv, hd, cos, False)
    kc, vc = _paged("bfloat16", n_pages, Hkv, ps, hd)
    q = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    w_tiles = K().tile_weight(w)
    K().gemm_rope_store(a, w, positions, row_req, tables, cos, sin, False, q, kc, vc, H, Hkv, hd, ps, w_tiles=w_tiles)
    # the same in two kernels
    qkv = torch.empty(T, (H + 2 * Hkv) * hd, dtype=torch.float32, device=DEV)
    K().gemm_tc(a, w, qkv, w_tiles=w_tiles)
    kc2, vc2 = _paged("bfloat16", n_pages, Hkv, ps, hd)
    q2 = torch.full_like(q, float("nan"))
    K().rope_store(qkv, positions, row_req, tables, cos, sin, False, q2, kc2, vc2, H, Hkv, hd, ps)
    assert K().gemm_tc_status(q.device) == 0
    for got, want, what in ((q, q2, "q"), (kc, kc2, "k pages"), (vc, vc2, "v pages")):
        got, want = got.float().cpu(), want.float().cpu()
        assert torch.equal(torch.isnan(got), torch.isnan(want)), f"{what}: other places were written"
        got, want = torch.nan_to_num(got), torch.nan_to_num(want)
        err = (got - want).abs().max().item()
        assert err <= 2.0 ** -7 * want.abs().max().item(), f"{what}: differs from the two-kernel path by {err}"   # one bfloat16 step
        assert (got != want).float().mean().item() < 0.02, f"{what}: too many values round differently"
    # no write without write_kv, and the same queries
    kc3, vc3 = _paged("bfloat16", n_pages, Hkv, ps, hd)
    q3 = torch.full_like(q, float("nan"))
    K().gemm_rope_store(a, w, positions, row_req, tables, cos, sin, False, q3, kc3, vc3, H, Hkv, hd, ps, write_kv=False,
                        w_tiles=w_tiles)
    assert torch.isnan(kc3.float()).all() and torch.isnan(vc3.float()).all()
    assert not torch.isnan(q3.float()).any() and torch.equal(q3, q), "queries must not depend on write_kv"


def test_l2_policy_of_streamed_loads_changes_no_result():
    """Weights of few-token products and keys/values of decode attention are loaded with the evict-first L2 policy:
    the same bits with the policy and without."""
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(8, 1032, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(520, 1032, generator=g) / 32).to(torch.bfloat16).to(DEV)
    outs, atts = [], []
    old = K().l2_streaming()
    try:
        for on in (True, False):
            K().l2_streaming(weights=on, keys_values=on)
            for tiles in (None, K().tile_weight(w)):
                out = torch.empty(8, 520, dtype=torch.float32, device=DEV)
                K().gemm_tc(a, w, out, w_tiles=tiles)
                outs.append(out)
            got, want = _attention_case("bfloat16", 8, 2, 64, 16, ctx_lens=[100, 700, 1, 300], q_lens=[1, 1, 1, 1], window=None,
                                        seed=5, fast=True)
            close(got, want, "bfloat16", "decode attention", bf16_tol=1e-2)
            atts.append(got)
    finally:
        K().l2_streaming(*old)
    assert K().l2_streaming() == old
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3]) and torch.equal(atts[0], atts[1])
    # a product that asks other memory into L2 while it runs (the weights of a product to come): the same bits,
    # whatever the size of that memory (less than a piece of 32 KB, pieces and a rest)
    for n in (1000, 32768 // 2 * 3 + 8):
        ahead = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
        out = torch.empty(8, 520, dtype=torch.float32, device=DEV)
        K().gemm_tc(a, w, out, w_tiles=K().tile_weight(w), ahead=ahead)
        assert torch.equal(out, outs[1])
    assert K().gemm_tc_status(a.device) == 0
    exact = a.double().cpu() @ w.double().cpu().T
    assert (outs[0].double().cpu() - exact).abs().max().item() <= 1e-4 * max(1.0, exact.abs().max().item())


def test_specialised_forms_of_the_few_token_product_give_the_same_bits():
    """The three forms a decode step runs (rotating [q; k; v] split over a cluster, added into the residual stream split
    over a cluster, stored unsplit) in kernels of their own against the kernel that holds every form."""
    g = torch.Generator().manual_seed(9)
    T, D, H, Hkv, hd, ps = 8, 2048, 32, 8, 64, 16
    a = (torch.randn(T, D, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w_qkv = (torch.randn((H + 2 * Hkv) * hd, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).to(DEV)
    w_o = (torch.randn(D, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).to(DEV)
    w_up = (torch.randn(4096, D, generator=g) / math.sqrt(D)).to(torch.bfloat16).to(DEV)
    tiles = [K().tile_weight(w) for w in (w_qkv, w_o, w_up)]
    x0 = torch.randn(T, D, generator=g).to(DEV)
    freq = 1.0 / (10000.0 ** (np.arange(hd // 2, dtype=np.float64) * 2 / hd))
    ang = np.arange(64, dtype=np.float64)[:, None] * freq[None]
    cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(DEV)
    sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(DEV)
    positions = torch.tensor([14, 15, 16, 17, 3, 40, 41, 0], dtype=torch.int32, device=DEV)
    row_req = torch.tensor([0, 0, 0, 0, 1, 2, 2, 3], dtype=torch.int32, device=DEV)
    tables = torch.tensor([[5, 2, -1], [7, -1, -1], [1, 0, 3], [8, -1, -1]], dtype=torch.int32, device=DEV)
    results = []
    old = K().specialised_products()
    try:
        for on in (True, False):
            K().specialised_products(on)
            kc, vc = _paged("bfloat16", 10, Hkv, ps, hd)
            q = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
            K().gemm_rope_store(a, w_qkv, positions, row_req, tables, cos, sin, False, q, kc, vc, H, Hkv, hd, ps, w_tiles=tiles[0])
            x = x0.clone()
            K().gemm_tc(a, w_o, x, accumulate=True, w_tiles=tiles[1])
            up = torch.full((T, 4096), float("nan"), dtype=torch.float32, device=DEV)
            K().gemm_tc(a, w_up, up, w_tiles=tiles[2])
            results.append((q, kc, vc, x, up))
    finally:
        K().specialised_products(old)
    assert K().gemm_tc_status(a.device) == 0
    for got, want, what in zip(results[0], results[1], ("q", "k pages", "v pages", "residual stream", "stored product")):
        assert torch.equal(torch.nan_to_num(got.float()), torch.nan_to_num(want.float())) and \
            torch.equal(torch.isnan(got.float()), torch.isnan(want.float())), what
    exact = x0.double().cpu() + a.double().cpu() @ w_o.double().cpu().T
    assert (results[0][3].double().cpu() - exact).abs().max().item() <= 1e-4 * max(1.0, exact.abs().max().item())
    exact = a.double().cpu() @ w_up.double().cpu().T
    assert (results[0][4].double().cpu() - exact).abs().max().item() <= 1e-4 * max(1.0, exact.abs().max().item())
