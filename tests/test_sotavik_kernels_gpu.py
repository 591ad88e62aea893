"""The kernels behind the latent-attention, recurrent and expert parts, each against plain float32
PyTorch of the same operation on the same (already rounded) inputs."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from supersonic_b200.csrc import ops as o
    return o


def rand(*shape, seed=0, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ---- latent attention ---------------------------------------------------------------------------------
def latent_case(lengths, new, H, dk, dv, seed):
    """A cache with ``lengths[b]`` rows per sequence of which the last ``new[b]`` are this step's tokens."""
    from supersonic_b200.cache import KvNeed, SequenceCache
    from supersonic_b200.engine import StepEntry, pack_step
    cache = SequenceCache({0: KvNeed(1, dk, None, value_dim=0)}, 4096, 2048, torch.bfloat16, DEV)
    slots = [cache.acquire() for _ in lengths]
    rows = [rand(n, dk, seed=seed + 10 * b, scale=0.5) for b, n in enumerate(lengths)]
    for s, n, k in zip(slots, lengths, new):
        cache.reserve(s, n - k)
        cache.advance(s, n - k)
    entries = [StepEntry(s, [0] * k) for s, k in zip(slots, new)]
    batch = pack_step(entries, [n - k for n, k in zip(lengths, new)], DEV)
    for s, k in zip(slots, new):
        cache.reserve(s, k)
    cache.sync()
    store, _, table, _ = cache.kv(0)
    for s, r in zip(slots, rows):
        for p in range(r.shape[0]):
            store[int(table[s, p // 64]), 0, p % 64] = r[p]
    q = rand(sum(new), H * dk, seed=seed + 1, scale=0.5)
    return cache, batch, store, table, q, rows


def latent_reference(q, rows, lengths, new, H, dk, dv, scale, sinks, window):
    out, at = [], 0
    for r, n, k in zip(rows, lengths, new):
        r = r.float()
        for t in range(k):
            pos = n - k + t
            lo = 0 if not window else max(0, pos - window + 1)
            qt = q[at + t].float().view(H, dk)
            s = (qt @ r[lo:pos + 1].T) * scale                                  # [H, keys]
            top = torch.maximum(s.max(dim=1).values, sinks) if sinks is not None else s.max(dim=1).values
            e = torch.exp(s - top[:, None])
            den = e.sum(1) + (torch.exp(sinks - top) if sinks is not None else 0.0)
            out.append(((e @ r[lo:pos + 1, :dv]) / den[:, None]).reshape(-1))
        at += k
    return torch.stack(out)


@pytest.mark.parametrize("H,dk,dv", [(6, 160, 128), (16, 288, 256), (3, 48, 32), (16, 576, 512), (40, 96, 64)])
@pytest.mark.parametrize("window", [None, 100])
def test_latent_attention_mma_prompts_and_decode(H, dk, dv, window):
    o = ops()
    scale = dk ** -0.5
    sinks = torch.linspace(-1.0, 2.0, H, device=DEV)
    # prompts that continue a cache, end inside a page, and a one-token prompt
    for lengths, new, splits in (([200, 65, 1, 130], [70, 65, 1, 3], 1), ([330, 64, 129], [1, 1, 1], 1),
                                 ([330, 64, 129], [1, 1, 1], 3), ([700, 5], [1, 1], 8)):
        cache, batch, store, table, q, rows = latent_case(lengths, new, H, dk, dv, seed=H + dk)
        T = sum(new)
        ref = latent_reference(q, rows, lengths, new, H, dk, dv, scale, sinks, window)
        plain = torch.empty(T, H * dv, dtype=torch.bfloat16, device=DEV)
        o.attention_plain(q, store, None, batch.pos, batch.slot_of_token, table, plain, H, 1, dk, 6, window, scale,
                          value_dim=dv, sinks=sinks)
        assert float((plain.float() - ref).abs().max()) < 0.02 * max(1.0, float(ref.abs().max()))
        for form in (0, 1, 2, 3):                                          # every layout of a block's warps
            out = torch.full((T, H * dv), 7.0, dtype=torch.bfloat16, device=DEV)
            assert o.latent_attention_mma_ok(q, store, out, H, dk, dv, 6)
            partial = torch.empty(T * H * splits * (dv + 2), device=DEV) if splits > 1 else None
            o.latent_attention_mma(q, store, batch.cu_new, batch.seq_start, batch.seq_slot, batch.slot_of_token, table, out,
                                   sinks, batch.max_new, H, dk, dv, 6, window, scale, splits, partial, form=form)
            assert float((out.float() - ref).abs().max()) < 0.02 * max(1.0, float(ref.abs().max())), (lengths, new, splits, form)


# ---- per-head and per-expert products ---------------------------------------------------------------
@pytest.mark.parametrize("T,H,K,N", [(1, 6, 64, 128), (133, 3, 128, 48), (70, 16, 24, 72)])
def test_head_products(T, H, K, N):
    o = ops()
    wide = rand(T, H * (K + 8), seed=1)
    x = wide.view(T, H, K + 8)[:, :, :K]                       # a view into wider rows
    w = rand(H, N, K, seed=2, scale=0.2)
    ref = torch.einsum("thk,hnk->thn", x.float(), w.float())
    for out_dtype in (torch.bfloat16, torch.float32):
        for fn in (o.head_linear_plain, o.head_gemm_mma):
            out = torch.zeros(T, H * N + 5, dtype=out_dtype, device=DEV)[:, : H * N].view(T, H, N)
            fn(x, w, out)
            assert float((out.float() - ref).abs().max()) < 0.02 * float(ref.abs().max()), fn.__name__
    xf, wf = x.float().contiguous(), w.float()
    out = torch.zeros(T, H, N, device=DEV)
    o.head_linear_plain(xf, wf, out)
    assert float((out - ref).abs().max()) < 1e-4 * float(ref.abs().max())


@pytest.mark.parametrize("T,top,E,K,N", [(1, 2, 5, 64, 40), (150, 3, 4, 128, 96), (64, 1, 7, 48, 200)])
def test_grouping_and_expert_products(T, top, E, K, N):
    o = ops()
    g = torch.Generator().manual_seed(T)
    expert_of = torch.rand(T, E, generator=g).argsort(1)[:, :top].int().contiguous().to(DEV)
    P = T * top
    max_tiles = o.expert_tiles_bound(P, E, 64)
    ints = [torch.zeros(n, dtype=torch.int32, device=DEV) for n in (E + 1, P, max_tiles, max_tiles, 1)]
    offsets, order, tile_expert, tile_row0, meta = ints
    o.group_by_expert(expert_of, E, 64, offsets, order, tile_expert, tile_row0, meta)
    flat = expert_of.view(-1).cpu()
    assert sorted(order.cpu().tolist()) == list(range(P))                       # a permutation of the pairs
    assert offsets.cpu().tolist() == [0] + torch.bincount(flat, minlength=E).cumsum(0).tolist()
    assert all(int(flat[p]) == e for e in range(E) for p in order[offsets[e]:offsets[e + 1]].cpu().tolist())
    assert int(meta[0]) == sum(-(-int(c) // 64) for c in torch.bincount(flat, minlength=E))
    x = rand(T, K, seed=3)
    w1 = rand(E, 2 * N, K, seed=4, scale=0.2)
    w2 = rand(E, K, N, seed=5, scale=0.2)
    pair_tok = torch.arange(P, device=DEV) // top
    e_of = expert_of.view(-1).long()
    gu = torch.einsum("pk,pnk->pn", x.float()[pair_tok], w1.float()[e_of])       # pair order
    act = torch.nn.functional.silu(gu[:, :N]) * gu[:, N:]
    inv = torch.empty(P, dtype=torch.long, device=DEV)
    inv[order.long()] = torch.arange(P, device=DEV)                             # pair -> sorted row
    groups = dict(order=order, offsets=offsets, tile_expert=tile_expert, tile_row0=tile_row0, meta=meta)
    for fn in (o.grouped_gemm_plain, o.grouped_gemm_mma):
        out = torch.zeros(P, 2 * N, dtype=torch.bfloat16, device=DEV)
        fn(x, order, top, w1, out, None, offsets, tile_expert, tile_row0, meta, max_tiles)
        assert float((out.float()[inv] - gu).abs().max()) < 0.02 * float(gu.abs().max()), fn.__name__
    z = torch.zeros(P, N, dtype=torch.bfloat16, device=DEV)
    o.grouped_gemm_mma(x, order, top, w1, z, None, offsets, tile_expert, tile_row0, meta, max_tiles, o.GG_SWIGLU)
    assert float((z.float()[inv] - act).abs().max()) < 0.03 * float(act.abs().max())
    zs = act[order.long()].bfloat16()                                           # sorted rows in, pair rows out
    want = torch.einsum("pn,pkn->pk", zs.float()[inv], w2.float()[e_of])
    for fn in (o.grouped_gemm_plain, o.grouped_gemm_mma):
        y = torch.zeros(P, K, device=DEV)
        fn(zs, None, 1, w2, y, order, offsets, tile_expert, tile_row0, meta, max_tiles)
        assert float((y - want).abs().max()) < 0.02 * float(want.abs().max()), fn.__name__
    pw = torch.rand(T, top, generator=g).to(DEV)
    res = torch.ones(T, K, device=DEV)
    o.expert_combine(res, want.contiguous(), pw, top)
    assert torch.allclose(res, 1 + (want.view(T, top, K) * pw[:, :, None]).sum(1), rtol=1e-5, atol=1e-5)


def test_table_router():
    o = ops()
    table = torch.tensor([[1, 2], [0, 3], [3, 1]], dtype=torch.int32, device=DEV)
    ids = torch.tensor([2, 0, 0, 1], dtype=torch.int32, device=DEV)
    e, w = torch.zeros(4, 2, dtype=torch.int32, device=DEV), torch.zeros(4, 2, device=DEV)
    o.route_table(ids, table, 4, e, w)
    assert e.cpu().tolist() == [[3, 1], [1, 2], [1, 2], [0, 3]] and torch.all(w == 0.5)


# ---- the recurrence ---------------------------------------------------------------------------------
def scan_reference(q, k, v, z, bias, tau, q_scale, S):
    out = []
    for t in range(q.shape[0]):
        a = torch.sigmoid(z[t] + bias).pow(1.0 / tau)
        S = a[:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t] * q_scale).reshape(-1))
    return torch.stack(out), S


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dv", [(2, 48, 32), (1, 256, 40), (3, 20, 72)])
def test_gated_linear_scan_in_one_go_and_in_chunks(dtype, H, d, dv):
    """Three sequences of unequal length from non-zero states: walked in one go, and cut into chunks of 64 and
    of 100 that run in parallel (the last chunk of every sequence is partial, one sequence has a single token)."""
    o = ops()
    lens = [300, 1, 130]
    T, tau = sum(lens), 3.0
    proj = rand(T, 2 * H * d + H * dv + 8, seed=1, dtype=dtype)
    z = rand(T, H * d, seed=2, scale=2.0, dtype=torch.float32)
    bias = rand(H * d, seed=3, dtype=torch.float32)
    state0 = rand(5, H * d * dv, seed=4, scale=0.3, dtype=torch.float32)
    cu = torch.tensor([0, 300, 301, 431], dtype=torch.int32, device=DEV)
    slots = torch.tensor([3, 0, 4], dtype=torch.int32, device=DEV)
    q_off, k_off, v_off = 8, 8 + H * d, 8 + 2 * H * d
    refs, ends = [], {}
    for b, s in enumerate(slots.tolist()):
        lo, hi = int(cu[b]), int(cu[b + 1])
        p = proj[lo:hi].double()
        r, S = scan_reference(p[:, q_off:q_off + H * d].view(-1, H, d), p[:, k_off:k_off + H * d].view(-1, H, d),
                              p[:, v_off:v_off + H * dv].view(-1, H, dv), z[lo:hi].double().view(-1, H, d),
                              bias.double().view(H, d), tau, d ** -0.5, state0[s].double().view(H, d, dv))
        refs.append(r)
        ends[s] = S.reshape(-1)
    ref = torch.cat(refs)
    for chunk in (0, 64, 100):
        state = state0.clone()
        out = torch.zeros(T, H * dv, device=DEV)
        n = -(-max(lens) // chunk) if chunk else 0
        sums = torch.empty(3 * n * H * d * dv, device=DEV) if chunk else None
        decays = torch.empty(3 * n * H * d, device=DEV) if chunk else None
        o.gated_linear_scan(proj, q_off, k_off, v_off, z.clone(), bias, tau, d ** -0.5, state, cu, slots, out, H, d, dv,
                            chunk=chunk, max_new=max(lens), sums=sums, decays=decays)
        assert float((out.double() - ref).abs().max()) < 2e-4 * max(1.0, float(ref.abs().max())), chunk
        for s, S in ends.items():
            assert float((state[s].double() - S).abs().max()) < 2e-4 * max(1.0, float(S.abs().max())), chunk
        assert torch.equal(state[1], state0[1]) and torch.equal(state[2], state0[2])      # other slots untouched


def test_head_norm_gate_stream_mix_and_scale():
    o = ops()
    T, H, dv = 9, 3, 40
    x = rand(T, H * dv, seed=1, dtype=torch.float32)
    w = rand(dv, seed=2)
    gate = rand(T, H * dv + 16, seed=3)[:, 16:]
    out = torch.zeros(T, H * dv, dtype=torch.bfloat16, device=DEV)
    o.head_norm_gate(x, w, 1e-5, gate, out, H, dv)
    xv = x.view(T, H, dv)
    ref = xv / torch.sqrt((xv * xv).mean(-1, keepdim=True) + 1e-5) * w.float() * torch.nn.functional.silu(gate.float()).view(T, H, dv)
    assert float((out.float().view(T, H, dv) - ref).abs().max()) < 0.02 * float(ref.abs().max())
    streams = rand(5, 7, 33, seed=4, dtype=torch.float32)
    wts = rand(5, seed=5, dtype=torch.float32)
    o.stream_mix(streams, wts, 3, streams[4])
    assert torch.allclose(streams[4], (streams[:3] * wts[:3, None, None]).sum(0), rtol=1e-6, atol=1e-6)
    y = streams[0].clone()
    o.scale_(y, 0.37)
    assert torch.allclose(y, streams[0] * 0.37)
