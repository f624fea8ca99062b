"""Teluzen through the framework (op table, ragged batches, block manager, scheduler, engine) against the plain oracle in
``teluzen_oracle.py``, on small random configurations.  These run on the CPU implementations of the ops;
``test_teluzen_gpu.py`` repeats the kernel-level and end-to-end comparisons on the CUDA kernels."""
import copy
import json

import pytest
import torch

import teluzen_oracle as oracle

F32 = 2e-4      # fp32 end to end against float64: rounding only


def make_engine(cfg, weights, dt=torch.float32, device="cpu", blocks=24, bs=8, max_batch=4, graphs=False):
    from llmctl_b200.serve.engine import InferenceEngine
    eng = InferenceEngine(copy.deepcopy(cfg), max_batch_size=max_batch, max_batch_tokens=blocks * bs, device=device,
                          kv_block_size=bs, num_kv_blocks=blocks, dtype=dt, kv_watermark=0.0, cuda_graphs=graphs)
    eng.model.load_state(weights)
    return eng


def small_cfg(per_layer=None, **kw):
    """``per_layer``: {layer index: mixer keys to override}, so that layers of one model differ in their sizes."""
    from llmctl_b200.models.teluzen import example_config
    cfg = example_config(**kw)
    for i, over in (per_layer or {}).items():
        m = cfg["layers"][i]["mixer"]
        for k, v in over.items():
            if k in ("size", "pool"):
                m["mask"][k] = v
            elif k == "rot_dims":
                m["rot"]["dims"] = v
            else:
                m[k] = v
    return cfg


def ref_logits(cfg, w, toks):
    return oracle.forward(cfg, w, toks)[0].float()


def run_cut(eng, sid, toks, cuts):
    """Feed ``toks`` in portions of the given sizes; returns logits of every position."""
    out, at = [], 0
    for c in cuts:
        assert eng.kv.allocate(sid, at + c)
        out.append(eng.forward_portions([eng.portion(sid, toks[at:at + c], at, list(range(c)))]))
        at += c
    assert at == len(toks)
    return torch.cat(out).float().cpu()


# ---- mechanisms alone ------------------------------------------------------------------------------------------
def test_sandwich_norm_ops_embedding_and_squared_relu():
    from llmctl_b200.ops import elementwise as E
    torch.manual_seed(0)
    y, x = torch.randn(6, 10), torch.randn(6, 10)
    wb, wn = torch.rand(10) + 0.5, torch.rand(10) + 0.5
    want_x = x + oracle.rms_norm(y, wb, 1e-3)
    h = E.sandwich_residual(y, x, wb, wn, 1e-3, torch.float32)
    assert torch.allclose(x, want_x, atol=1e-6) and torch.allclose(h, oracle.rms_norm(want_x, wn, 1e-3), atol=1e-6)
    hb, h32 = E.sandwich_residual(y.clone(), x.clone() - oracle.rms_norm(y, wb, 1e-3), wb, wn, 1e-3, torch.bfloat16, want_fp32=True)
    assert hb.dtype == torch.bfloat16 and torch.allclose(h32, h, atol=1e-6) and torch.equal(hb, h32.to(torch.bfloat16))
    assert E.sandwich_residual(y, x, wb, None, 1e-3, torch.float32) is None
    assert torch.allclose(x, want_x + oracle.rms_norm(y, wb, 1e-3), atol=1e-6)
    assert torch.allclose(E.rmsnorm_rows(x, torch.tensor([4, 1]), wn, 1e-3, torch.float32), oracle.rms_norm(x[[4, 1]], wn, 1e-3), atol=1e-6)
    # eps sits inside the root: a zero row stays zero instead of dividing by zero
    assert torch.equal(E.rmsnorm_rows(torch.zeros(1, 10), None, wn, 1e-3, torch.float32), torch.zeros(1, 10))
    table, pos = torch.randn(9, 4), torch.randn(30, 4)
    got = E.embed_positions(torch.tensor([3, 3, 8]), torch.tensor([0, 29, 5], dtype=torch.int32), table, pos)
    assert torch.equal(got, table[[3, 3, 8]] + pos[[0, 29, 5]])
    z = torch.linspace(-3, 3, 13)
    assert torch.equal(E.relu_squared(z), torch.relu(z) ** 2)


def test_rotary_spectrum_matches_oracle():
    from llmctl_b200.ops.elementwise import rope_frequencies
    for dims, base, sc in ((8, 10000.0, None), (16, 5e5, {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}),
                           (2, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 2.0}),
                           (6, 3000.0, {"factor": 3.0, "original": 40, "fast": 8.0, "slow": 0.5})):
        f, m = rope_frequencies(dims, base, sc)
        fo, mo = oracle.rotary_spectrum(dims, base, sc)
        assert torch.allclose(f.double(), fo, rtol=1e-6, atol=0) and abs(m - mo) < 1e-7


@pytest.mark.parametrize("H,G,d,e,rot", [(4, 2, 8, 6, 4), (3, 3, 6, 6, 6), (6, 1, 4, 10, 0), (2, 2, 10, 3, 2)])
def test_projection_postprocessing_and_cache_append(H, G, d, e, rot):
    """Bias, norm over the WHOLE q / k projection (not per head), rotation of the first ``rot`` numbers of every head as
    interleaved pairs, value mixing; q, the cache rows and v_first against the oracle's pieces."""
    from llmctl_b200.ops import window_attention as W
    from llmctl_b200.ops.elementwise import rope_frequencies
    torch.manual_seed(1)
    T, bs, P = 7, 4, 3
    PS = W.pooled_rows_per_page(bs, P)
    Nq, Nk, Nv = H * d, G * d, G * e
    qkv, bias = torch.randn(T, Nq + Nk + Nv), torch.randn(Nq + Nk + Nv)
    qn, kn = torch.rand(Nq) + 0.5, torch.rand(Nk) + 0.5
    sc = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
    f, mult = rope_frequencies(rot, 500.0, sc) if rot else (torch.zeros(1), 1.0)
    pos = torch.tensor([0, 1, 2, 40, 41, 999, 5], dtype=torch.int32)
    slots = torch.tensor([0, 1, 2, 9, 10, -1, 7])
    cache = torch.zeros(5, bs + PS, Nk + Nv)
    vf = torch.zeros(T, Nv)
    q = W.window_qkv_write(qkv, bias, qn, kn, H, G, d, e, rot, f, mult, 1e-5, pos, slots, cache, bs, vf, 1, None)
    full = (qkv + bias).double()
    qo = oracle.rms_norm(full[:, :Nq], qn.double(), 1e-5).reshape(T, H, d)
    ko = oracle.rms_norm(full[:, Nq:Nq + Nk], kn.double(), 1e-5).reshape(T, G, d)
    if rot:
        qo = oracle.rotate_pairs(qo, pos, rot, 500.0, sc)
        ko = oracle.rotate_pairs(ko, pos, rot, 500.0, sc)
    assert torch.allclose(q.double(), qo.reshape(T, Nq), atol=1e-5)
    rows = (slots // bs) * (bs + PS) + slots % bs
    ok = slots >= 0
    flat = cache.view(-1, Nk + Nv)
    assert torch.allclose(flat[rows[ok], :Nk].double(), ko.reshape(T, Nk)[ok], atol=1e-5)
    assert torch.allclose(flat[rows[ok], Nk:].double(), full[ok, Nq + Nk:], atol=1e-6) and torch.allclose(vf.double(), full[:, Nq + Nk:], atol=1e-6)
    # a later layer blends with the first layer's values; the blend is what it caches
    lam = torch.tensor([0.3])
    cache2 = torch.zeros_like(cache)
    qkv2 = torch.randn(T, Nq + Nk + Nv)
    W.window_qkv_write(qkv2, bias, qn, kn, H, G, d, e, rot, f, mult, 1e-5, pos, slots, cache2, bs, vf, 2, lam)
    want = 0.7 * (qkv2 + bias)[:, Nq + Nk:] + 0.3 * vf
    assert torch.allclose(cache2.view(-1, Nk + Nv)[rows[ok], Nk:], want[ok], atol=1e-6)
    assert float(cache.view(-1, Nk + Nv)[[3, bs, bs + 1]].abs().max()) == 0.0      # rows nobody was given stay untouched


def _fill_cache(k, v, bs, P, table, pages):
    """Cache rows of one sequence (k [n, G, d], v [n, G, e]) written through the product's own append + pool ops."""
    from llmctl_b200.ops import window_attention as W
    n, G, d = k.shape
    e = v.shape[2]
    PS = W.pooled_rows_per_page(bs, P)
    cache = torch.zeros(pages, bs + PS, G * (d + e))
    flat = cache.view(-1, G * (d + e))
    tb = torch.tensor([table], dtype=torch.int32)
    for j in range(n):
        flat[table[j // bs] * (bs + PS) + j % bs] = torch.cat([k[j].reshape(-1), v[j].reshape(-1)])
    pos = torch.arange(n, dtype=torch.int32)
    slots = torch.tensor([table[j // bs] * bs + j % bs for j in range(n)])
    W.window_pool_update(cache, pos, slots, torch.zeros(n, dtype=torch.int32), tb, bs, P)
    return cache, tb


@pytest.mark.parametrize("S,P,bs", [(10, 4, 8), (7, 3, 8), (5, 1, 4), (9, 12, 8), (16, 8, 8), (1, 2, 4)])
def test_window_and_pooled_blocks_against_oracle(S, P, bs):
    """Every query position of a 70-token sequence, one at a time (as in decoding) and in tiles: windows and pools that
    do not divide the page, a pool larger than a page, a pool of one (every token before the window), a window of one."""
    from llmctl_b200.ops import window_attention as W
    from llmctl_b200.serve.ragged import Portion, RaggedBatch
    torch.manual_seed(2)
    n, H, G, d, e = 70, 4, 2, 6, 5
    k, v, q = torch.randn(n, G, d), torch.randn(n, G, e), torch.randn(n, H, d)
    temp, talk = torch.rand(H) + 0.5, torch.eye(H) + 0.3 * torch.randn(H, H)
    pages = (n + bs - 1) // bs
    table = torch.randperm(pages + 3).tolist()[:pages]
    cache, _ = _fill_cache(k, v, bs, P, table, pages + 3)
    ref = oracle.attend(q.double(), k.double(), v.double(), S, P, 0.4, temp.double(), talk.double()).reshape(n, H * e)
    whole = RaggedBatch([Portion(1, [0] * n, 0, [], table)], bs, torch.device("cpu"))
    got = W.pooled_window_attention(q.reshape(n, H * d), cache, whole.block_tables, whole.tiles(16), 16, whole.positions, temp, talk,
                                    0.4, H, G, d, e, S, P, bs, torch.float32)
    assert torch.allclose(got.double(), ref, atol=1e-5)
    for i in (0, S - 1, S, S + P - 1, S + P, n - 1):
        if i >= n:
            continue
        one = RaggedBatch([Portion(1, [0], i, [], table)], bs, torch.device("cpu"))
        g1 = W.pooled_window_attention(q[i].reshape(1, H * d), cache, one.block_tables, one.tiles(16), 1, one.positions, temp, talk,
                                       0.4, H, G, d, e, S, P, bs, torch.float32)
        assert torch.allclose(g1[0].double(), ref[i], atol=1e-5), f"position {i}"


def _decisive(n, far, d, e, G=1):
    """Keys and values in which token ``far`` alone matches the query direction strongly."""
    k, v = 0.05 * torch.randn(n, G, d), torch.randn(n, G, e)
    k[far, :, 0] = 12.0
    q = torch.zeros(1, G, d)
    q[..., 0] = 12.0
    return q, k, v


def test_window_edge_and_pool_edge_decide():
    """One token carries a key that dominates every softmax it takes part in.  Just inside the window it is the output;
    one step later it has left the window and, until its block is complete AND wholly before the window, it is not
    seen at all; after that it is seen through its block's mean."""
    from llmctl_b200.ops import window_attention as W
    from llmctl_b200.serve.ragged import Portion, RaggedBatch
    torch.manual_seed(3)
    S, P, bs, d, e = 9, 4, 8, 4, 3
    for far in (0, 5, 7, 8, 22, 23, 24, 63, 64):
        n = far + S + 2 * P + 2
        q, k, v = _decisive(n, far, d, e)
        pages = (n + bs - 1) // bs
        table = torch.randperm(pages + 2).tolist()[:pages]
        cache, _ = _fill_cache(k, v, bs, P, table, pages + 2)
        block_end = far // P * P + P - 1
        for i in range(far, n):
            b = RaggedBatch([Portion(1, [0], i, [], table)], bs, torch.device("cpu"))
            out = W.pooled_window_attention(q.reshape(1, d), cache, b.block_tables, b.tiles(16), 1, b.positions, None, None, 1.0,
                                            1, 1, d, e, S, P, bs, torch.float32)[0]
            if i - far < S:
                assert torch.allclose(out, v[far, 0], atol=1e-3), f"far {far}: inside the window at {i}"
            elif block_end <= i - S:
                blk = v[far // P * P: far // P * P + P, 0].mean(0)
                assert torch.allclose(out, blk, atol=1e-3), f"far {far}: through its block at {i}"
            else:
                assert (out - v[far, 0]).abs().max() > 0.05 and (out.abs() < 4).all(), f"far {far}: must be invisible at {i}"
            want = oracle.attend(q.double().expand(i + 1, 1, d), k[:i + 1].double(), v[:i + 1].double(), S, P, 1.0, None, None)[i, 0]
            assert torch.allclose(out.double(), want, atol=1e-5)


def test_head_temperature_weight_mixing_and_value_groups():
    """Temperatures scale scores per head; the mixing acts on NORMALISED weights (rows of ``talk`` need not sum to one);
    a mixed head applies its weights to its OWN key/value head's values."""
    from llmctl_b200.ops import window_attention as W
    from llmctl_b200.serve.ragged import Portion, RaggedBatch
    torch.manual_seed(4)
    n, H, G, d, e, bs = 13, 4, 2, 3, 2, 4
    k, v, q = torch.randn(n, G, d), torch.randn(n, G, e), torch.randn(n, H, d)
    table = [2, 0, 3, 1]
    cache, _ = _fill_cache(k, v, bs, 2, table, 4)
    b = RaggedBatch([Portion(1, [0] * n, 0, [], table)], bs, torch.device("cpu"))
    temp = torch.tensor([0.5, 2.0, 1.0, 3.0])
    talk = torch.tensor([[0.0, 0.0, 0.0, 2.0], [0.5, 0.5, 0.0, 0.0], [0.0, 0.0, 1.0, 0.0], [1.0, -1.0, 1.0, 0.5]])
    got = W.pooled_window_attention(q.reshape(n, -1), cache, b.block_tables, b.tiles(16), 16, b.positions, temp, talk, 0.7, H, G, d, e,
                                    0, 0, bs, torch.float32).view(n, H, e)
    # by hand for the last position: head 0 uses 2 x head 3's weights on the values of ITS group (group 0)
    s3 = (q[-1, 3] @ k[:, 1].T) * 0.7 * 3.0
    assert torch.allclose(got[-1, 0], 2.0 * torch.softmax(s3, -1) @ v[:, 0], atol=1e-5)
    ref = oracle.attend(q.double(), k.double(), v.double(), None, None, 0.7, temp.double(), talk.double())
    assert torch.allclose(got.double(), ref, atol=1e-5)


@pytest.mark.parametrize("top,E,shared", [(1, 4, True), (2, 5, True), (3, 3, False), (4, 4, True)])
def test_feed_forwards_against_oracle(top, E, shared):
    from llmctl_b200.models.ffn import GatedExpertMoE, SquaredReluMLP
    torch.manual_seed(5)
    W, ff, sf = 12, 6, 10
    mlp = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": ff}, "shared": {"ff": sf} if shared else None}
    p = {"router": torch.randn(E, W)}
    for n in [f"e{e}." for e in range(E)] + (["shared."] if shared else []):
        f_ = sf if n == "shared." else ff
        p.update({n + "gate": torch.randn(f_, W) / 3, n + "up": torch.randn(f_, W) / 3, n + "down": torch.randn(W, f_) / 3})
    m = GatedExpertMoE(W, E, top, ff, sf if shared else None, torch.float32, "cpu", scale_input=False, softmax_scores=2, shared_gate=False)
    m.load(lambda k: p[k], "")
    x = torch.randn(9, W)
    assert torch.allclose(m(x, x).double(), oracle.moe_ff(x.double(), mlp, {k: v.double() for k, v in p.items()}, ""), atol=1e-5)
    # the weights of the chosen experts sum to one whatever the other logits are
    from llmctl_b200.ops import moe as M
    ids, wts, _, _ = M.route(x, p["router"], top, softmax=2)
    oi, ow = oracle.route(x.double(), p["router"].double(), top)
    assert torch.equal(ids.long(), oi) and torch.allclose(wts.double(), ow, atol=1e-6) and torch.allclose(wts.sum(-1), torch.ones(9))
    d = SquaredReluMLP(W, 7, torch.float32, "cpu")
    pd = {"up": torch.randn(7, W), "down": torch.randn(W, 7)}
    d.load(lambda k: pd[k], "")
    assert torch.allclose(d(x, x).double(), oracle.dense_ff(x.double(), {k: v.double() for k, v in pd.items()}, ""), atol=1e-4)


# ---- whole models ----------------------------------------------------------------------------------------------
CONFIGS = {
    "default": dict(),
    "odd_sizes": dict(width=40, heads=6, kv_heads=3, dim=6, vdim=5, rot_dims=2, window=7, pool=3, ff=33, experts=3, top=1, expert_ff=9,
                      shared_ff=None, pattern="MD-M", v_mix="1011", yarn=False),
    "every_head_its_own": dict(heads=3, kv_heads=3, dim=4, vdim=4, rot_dims=4, window=9, pool=1, pattern="DM", v_mix="11"),
    "one_kv_head": dict(heads=5, kv_heads=1, dim=6, vdim=9, rot_dims=6, window=20, pool=12, experts=4, top=4, pattern="MM", v_mix="00"),
    "window_longer_than_prompt": dict(window=200, pool=5, pattern="D-", v_mix="01"),
    "layers_differ": dict(pattern="DMD", v_mix="101",
                          per_layer={0: dict(heads=2, kv_heads=1, dim=10, size=6, pool=2, rot_dims=10, scale=0.2),
                                     1: dict(heads=8, kv_heads=4, dim=4, size=11, pool=5, rot_dims=2),
                                     2: dict(heads=4, kv_heads=2, dim=6, vdim=6, size=1, pool=1)}),
}


def _cfg(name):
    kw = dict(CONFIGS[name])
    per = kw.pop("per_layer", None)
    cfg = small_cfg(per, **kw)
    if name == "layers_differ":        # layers that mix values must agree on the value sizes: layer 2 mixes with layer 0
        cfg["layers"][0]["mixer"].update(kv_heads=2, vdim=5)
        cfg["layers"][2]["mixer"].update(kv_heads=2, vdim=5)
    return cfg


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_layer_trace(name):
    cfg = _cfg(name)
    w = oracle.random_weights(cfg, seed=11)
    toks = torch.randint(0, cfg["vocab"], (45,), generator=torch.Generator().manual_seed(1)).tolist()
    ref, tr = oracle.forward(cfg, w, toks)
    eng = make_engine(cfg, w)
    assert eng.kv.allocate(1, len(toks))
    mine = []
    got = eng.forward_portions([eng.portion(1, toks, 0, list(range(len(toks))))], layer_trace=mine)
    assert len(mine) == len(tr)
    for i, (a, b) in enumerate(zip(mine, tr)):
        assert torch.allclose(a.double(), b, atol=F32), f"residual stream differs after layer {i}"
    assert torch.allclose(got.double(), ref, atol=F32)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_portions_and_decode_agree(name):
    """Token-by-token decoding, portions down to two tokens cut inside pages, windows and pooled blocks, and one whole
    prompt give the oracle's logits at every position (pages of 8, prompt over several pages)."""
    cfg = _cfg(name)
    w = oracle.random_weights(cfg, seed=12)
    toks = torch.randint(0, cfg["vocab"], (61,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = ref_logits(cfg, w, toks)
    eng = make_engine(cfg, w)
    for sid, cuts in enumerate(([1] * 61, [2, 5, 8, 1, 17, 2, 2, 16, 3, 1, 1, 1, 1, 1], [7, 54], [60, 1]), start=1):
        got = run_cut(eng, sid, toks, cuts)
        assert torch.allclose(got, ref, atol=F32), f"cuts {cuts[:4]}..."
        eng.kv.free(sid)


def test_value_mixing_layers_need_equal_value_sizes():
    from llmctl_b200.models.teluzen import TeluzenConfig
    cfg = small_cfg({1: dict(vdim=7)}, pattern="DD", v_mix="11")
    with pytest.raises(ValueError):
        TeluzenConfig.from_dict(cfg)
    TeluzenConfig.from_dict(small_cfg({1: dict(vdim=7)}, pattern="DD", v_mix="10"))


def test_unequal_batch_matches_each_alone_and_pages_are_reused():
    """Four live requests of unequal length advance in mixed batches (portions next to single tokens, some skipping a
    step) in a pool that only holds them because finished requests give their pages (and pooled rows) back."""
    cfg = small_cfg(window=10, pool=3)
    w = oracle.random_weights(cfg, seed=13)
    g = torch.Generator().manual_seed(3)
    lens = [50, 9, 33, 1, 26, 40, 17]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    refs = [ref_logits(cfg, w, r) for r in reqs]
    eng = make_engine(cfg, w, blocks=18, bs=8)          # 144 token slots < sum(lens) = 176
    waiting, live, done, step = list(range(len(reqs))), {}, 0, 0
    owners_of_block = {}
    while waiting or live:
        while waiting and len(live) < 4 and eng.kv.free_blocks * 8 >= lens[waiting[0]] + 8:
            live[waiting.pop(0)] = 0
        portions, owners = [], []
        for k, (i, at) in enumerate(sorted(live.items())):
            if (step + i) % 5 == 4:
                continue                                  # left out of this step
            n = min([1, 2, 11, 1, 5][(step + k) % 5], lens[i] - at) if at else min(3 + 4 * k, lens[i])
            assert eng.kv.allocate(100 + i, at + n)
            for blk in eng.kv.block_table(100 + i):
                owners_of_block.setdefault(blk, set()).add(i)
            portions.append(eng.portion(100 + i, reqs[i][at:at + n], at, list(range(n))))
            owners.append((i, at, n))
        if portions:
            lg = eng.forward_portions(portions)
            o = 0
            for i, at, n in owners:
                assert torch.allclose(lg[o:o + n], refs[i][at:at + n], atol=F32), f"request {i} at {at} (+{n}) in step {step}"
                o += n
                live[i] = at + n
                if at + n == lens[i]:
                    eng.kv.free(100 + i)
                    del live[i]
                    done += 1
        step += 1
        assert step < 400
    assert done == len(reqs) and eng.kv.free_blocks == 18
    assert sum(len(v) > 1 for v in owners_of_block.values()) >= 4, "pages were not handed out again"


def test_long_decode_through_engine_scheduler_is_greedy_consistent():
    """Greedy generation through ``InferenceEngine.generate`` (scheduler, block growth, batched decode of unequal
    requests) well past the window and several pooled blocks: every generated token is the oracle's argmax."""
    cfg = small_cfg(window=9, pool=4, pattern="DMD", v_mix="011")
    w = oracle.random_weights(cfg, seed=14)
    eng = make_engine(cfg, w, blocks=40, bs=8)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 19, 1)]
    outs = eng.generate(prompts, max_tokens=60, temperature=0.0)
    assert sum(len(o) for o in outs) >= 100 and max(len(o) for o in outs) == 60       # a sequence may stop early at the end token
    for p, o in zip(prompts, outs):
        ref = ref_logits(cfg, w, p + o)
        top2 = ref.topk(2, -1).values
        for k, tok in enumerate(o):
            row = len(p) + k - 1
            if top2[row, 0] - top2[row, 1] > 1e-3:          # skip near ties
                assert tok == int(ref[row].argmax()), f"token {k} of prompt len {len(p)}"
    assert eng.kv.free_blocks == 40


def test_config_reader_registry_and_trace_replay(tmp_path):
    """config.json + model.safetensors -> registry -> engine; the replayer admits requests at their first entry, lets
    one skip a step, frees pages at ``end`` and writes logits in entry order; freed pages serve new requests."""
    from safetensors.torch import save_file
    from llmctl_b200.models.config import resolve_model
    from llmctl_b200.models.teluzen import TeluzenConfig
    from llmctl_b200.serve.replay import TraceReplayer
    cfg = small_cfg(pattern="DM", window=48, pool=6)
    w = oracle.random_weights(cfg, seed=16)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    c = resolve_model(tmp_path)
    assert isinstance(c, TeluzenConfig) and c.layers[1].mixer.v_mix and c.layers[0].mixer.window == 48 and c.layers[1].mlp["kind"] == "moe"
    bad = copy.deepcopy(cfg)
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        TeluzenConfig.from_dict(bad)
    a = list(range(3, 80))
    b = list(range(40, 50))
    ra, rb = ref_logits(cfg, w, a), ref_logits(cfg, w, b)
    rp = TraceReplayer(str(tmp_path), "float32", max_tokens=192, device="cpu")      # three pages of 64: a holds two, b one
    l0 = rp.step({"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []})
    assert torch.allclose(l0, torch.stack([ra[0], ra[69], rb[1]]), atol=F32)
    assert rp.step({"step": 1, "entries": [{"id": "b", "tokens": b[2:9], "want": []}], "end": []}) is None
    l2 = rp.step({"step": 2, "entries": [{"id": "b", "tokens": b[9:], "want": [0]}, {"id": "a", "tokens": a[70:], "want": [6]}], "end": ["a", "b"]})
    assert torch.allclose(l2, torch.stack([rb[9], ra[76]]), atol=F32)
    assert rp.engine.kv.free_blocks == 3 and not rp.live
    l3 = rp.step({"step": 3, "entries": [{"id": "c", "tokens": a, "want": [76]}, {"id": "d", "tokens": b, "want": [9]}], "end": ["c"]})
    assert torch.allclose(l3, torch.stack([ra[76], rb[9]]), atol=F32)


def test_bfloat16_serving_precision_is_close_to_oracle():
    cfg = small_cfg()
    w = oracle.random_weights(cfg, seed=17)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(6)).tolist()
    ref = ref_logits(cfg, w, toks)
    eng = make_engine(cfg, w, dt=torch.bfloat16)
    got = run_cut(eng, 1, toks, [25] + [1] * 15)
    err = (got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()
    assert err < 0.05, err
