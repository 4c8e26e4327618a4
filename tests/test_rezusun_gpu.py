"""The Rezusun design on the GPU against its plain restatement (tests/plain_rezusun.py):
each mechanism alone, then whole models through the step function, the cache, the scheduler
and the generation entry point, in float32 and bfloat16."""

import os
import tempfile

import numpy as np
import pytest
import torch

import plain_rezusun as R
import tiny_rezusun as tiny

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 4e-2}
# whole models here are eleven sublayers deep with weights of unit gain: bfloat16 rounding adds up to more
# than in one part alone (and is measured as a root mean square, see _logit_err); float32 stays the sharp comparison
TOL_MODEL = {"float32": 3e-5, "bfloat16": 9e-2}


def _ctx(dtype, max_positions=512):
    from kv_cache_optimization_for_llm_b200.parts import BuildContext
    dev = torch.device("cuda:0")
    return BuildContext(dtype=DT[dtype], device=dev, max_positions=max_positions,
                        status=torch.zeros(1, dtype=torch.int32, device=dev))


def _w(rng, shape, std=0.3, mean=0.0):
    """A tensor that bfloat16 holds exactly, and its float64 copy."""
    t = torch.as_tensor(mean + rng.normal(size=shape) * std, dtype=torch.float32).to(torch.bfloat16)
    return t, t.float().numpy().astype(np.float64)


def _rel(got, ref):
    return np.abs(got.detach().float().cpu().numpy().astype(np.float64) - ref).max() / np.abs(ref).max()


class _Manager:
    """Stands in for the cache manager when a part runs alone: request r sits in slot
    ``slots[r]`` and owns the pages ``tables[r]``."""

    def __init__(self, tables, slots):
        self.tables, self.slots = tables, slots

    def slot_of(self, rid):
        return self.slots[rid]

    def block_table(self, rid, g):
        return self.tables[rid]


def _builder(ctx, max_pages=64):
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder
    return BatchBuilder(1024, 8, [max_pages], ctx.device, ctx.status)


def _make(family, kind, params, weights, ctx, wspecs=None):
    """Builds a part from float tensors the way the model does (kinds decide the precision)."""
    from kv_cache_optimization_for_llm_b200.parts import lookup
    from kv_cache_optimization_for_llm_b200.weights.loader import to_compute
    cls = lookup(family, kind)
    specs = cls.weight_specs(params)
    assert set(specs) == set(weights), (sorted(specs), sorted(weights))
    dev = {}
    for role, t in weights.items():
        assert tuple(t.shape) == tuple(specs[role].shape), (role, t.shape, specs[role].shape)
        dev[role] = to_compute(t, specs[role], ctx.dtype, ctx.device)
    return cls(params, dev, ctx)


# --------------------------------------------------------------------------- norms and feed-forward

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [40, 333])
def test_post_norm_add_pre_norm_in_one_kernel(dtype, H):
    """residual += scale * LN_b(branch + bias), then LN(residual): against the plain formulas, for
    every row and for picked rows, with layer norms, RMS norms and no post norm."""
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(H)
    T = 7
    res0 = rng.normal(size=(T, H)) * 2 + 0.5
    delta_t, delta = _w(rng, (T, H), 1.5, 0.7)
    bias = rng.normal(size=H)
    wb, ws, w = 1 + 0.2 * rng.normal(size=H), 0.3 * rng.normal(size=H), 1 + 0.2 * rng.normal(size=H)
    f32 = lambda a: torch.as_tensor(a, dtype=torch.float32).cuda()
    d64 = lambda t: t.cpu().numpy().astype(np.float64)
    res0 = d64(f32(res0))
    bias64, wbs64, w64 = d64(f32(bias)), d64(f32(wb) * f32(ws)), d64(f32(w))
    for post, pre in (("layer", "layer"), ("rms", "layer"), ("layer", "rms"), (None, "layer")):
        resid = f32(res0)
        if post is None:
            pending, add = delta_t.to(DT[dtype]).cuda(), delta
        else:
            pending = ops.PostNormed(delta_t.to(DT[dtype]).cuda(), f32(bias), post, f32(wb) * f32(ws), 1e-5)
            normed = R.layer_norm(delta + bias64, wbs64, 1e-5) if post == "layer" else R.rms_norm(delta + bias64, wbs64, 1e-5)
            add = normed
        want_res = res0 + add
        want = R.layer_norm(want_res, w64, 1e-5) if pre == "layer" else R.rms_norm(want_res, w64, 1e-5)
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
        picked = ops.add_norm(resid, pending, pre, f32(w), 1e-5, DT[dtype], rows)
        assert np.array_equal(d64(resid), res0), "picking rows must leave the residual alone"
        assert _rel(picked, want[[5, 0, 5]]) < TOL[dtype]
        out = ops.add_norm(resid, pending, pre, f32(w), 1e-5, DT[dtype])
        assert _rel(out, want) < TOL[dtype], (post, pre)
        assert _rel(resid, want_res) < 3e-6, "the residual is float32 in both precisions"
        if post is not None:
            assert _rel(pending.materialize(), add) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_dense_feed_forward_alone(dtype):
    rng = np.random.default_rng(1)
    ctx = _ctx(dtype)
    H, I, T = 56, 72, 9
    wt, w64 = {}, {}
    for role, name, shape in (("gate", "gate", (I, H)), ("up", "up", (I, H)), ("down", "down", (H, I)),
                              ("gate_bias", "gate.b", (I,)), ("up_bias", "up.b", (I,)), ("down_bias", "down.b", (H,))):
        wt[role], w64[name] = _w(rng, shape, 0.3)
    ff = _make("feed_forward", "gated_dense", {"hidden_size": H, "intermediate_size": I, "activation": "gelu_tanh",
                                               "bias": True}, wt, ctx)
    x, x64 = _w(rng, (T, H), 1.0)
    ref = R.dense_feed_forward(x64, w64, "")
    assert _rel(ff.forward(x.to(DT[dtype]).cuda(), None), ref) < TOL[dtype]
    y, b = ff.forward(x.to(DT[dtype]).cuda(), None, bias_out=True)
    assert _rel(y.float() + b, ref) < TOL[dtype]


# --------------------------------------------------------------------------- the mixers alone

def _run_in_steps(mixer, ctx, x, steps, page=8, state_slots=3):
    """Feeds requests through a mixer alone.  ``x``: request -> its inputs [T, H] (compute type, on
    the device); ``steps``: a list of steps, each a list of (request, number of tokens).  Requests
    sit in slots and pages of their own (slot = request + 1 so that slot 0 stays untouched).
    Returns request -> outputs [T, H]."""
    from kv_cache_optimization_for_llm_b200.cache.specs import PagedKVBinding, PagedKVSpec, SlotStateBinding
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    spec = mixer.cache_spec()
    n_req = len(x)
    pages_each = -(-max(t.shape[0] for t in x.values()) // page)
    # pages are dealt out backwards and interleaved, so that a request's pages are neither in order nor adjacent
    tables = {r: [n_req * pages_each - 1 - (i * n_req + r) for i in range(pages_each)] for r in x}
    slots = {r: (r + 1) % (state_slots + 1) for r in x}
    if isinstance(spec, PagedKVSpec):
        store = torch.zeros((spec.planes, n_req * pages_each + 1, spec.num_kv_heads, page, spec.head_dim),
                            dtype=ctx.dtype, device=ctx.device)
        binding = PagedKVBinding(k=store[0], v=store[1] if spec.planes > 1 else None, group=0, page_size=page)
    else:
        # the states start full of rubbish: a request that starts at position 0 must not read them
        state = torch.full((state_slots + 1,) + tuple(spec.shape), 7.5, dtype=spec.dtype, device=ctx.device)
        binding = SlotStateBinding(state=state)
    builder = _builder(ctx)
    at = {r: 0 for r in x}
    outs = {r: [] for r in x}
    for step in steps:
        entries = [StepEntry(r, [0] * n, at[r], ()) for r, n in step]
        batch = builder.build(entries, _Manager(tables, slots))
        order = sorted(range(len(step)), key=lambda i: (len(step) > 1 and any(m == 1 for _, m in step)
                                                         and any(m != 1 for _, m in step) and step[i][1] != 1, i))
        rows = torch.cat([x[step[i][0]][at[step[i][0]]:at[step[i][0]] + step[i][1]] for i in order]).contiguous()
        y = mixer.forward(rows, batch, binding)
        t = 0
        for i in order:
            r, n = step[i]
            outs[r].append(y[t:t + n].float().cpu())
            t += n
            at[r] += n
    assert int(ctx.status.item()) == 0
    return {r: torch.cat(o) for r, o in outs.items()}


def _general_weights(rng, H, heads, dim, rank):
    hd = heads * dim
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (
            ("r", "r", (hd, H), 0.3, 0), ("k", "k", (hd, H), 0.3, 0), ("v", "v", (hd, H), 0.3, 0),
            ("g", "g", (hd, H), 0.3, 0), ("a", "a", (hd, H), 0.3, 0), ("a_bias", "a.b", (hd,), 0.5, 0),
            ("w1", "w1", (rank, H), 0.3, 0), ("w2", "w2", (hd, rank), 0.6, 0), ("w0", "w0", (hd,), 1.0, 0),
            ("norm", "norm", (hd,), 0.2, 1), ("o", "o", (H, hd), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rank", [(2, 16, 6), (3, 20, 9), (1, 64, 16), (2, 128, 8), (5, 4, 1)])
def test_general_delta_alone_in_portions_and_beside_another_request(dtype, heads, dim, rank):
    rng = np.random.default_rng(dim)
    ctx = _ctx(dtype)
    H = 40
    wt, w64 = _general_weights(rng, H, heads, dim, rank)
    mx = {"heads": heads, "dim": dim}
    mixer = _make("mixer", "general_delta", {"hidden_size": H, "heads": heads, "dim": dim, "decay_rank": rank,
                                             "eps": 1e-5}, wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((45, 19)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), R.general_delta(x64, w64, "", mx, 1e-5)
    # whole, then the same requests cut: portions of 17, 2, 1 and 16 + 9 tokens beside single tokens
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 45)], [(1, 19)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 17), (1, 1)], [(0, 2), (1, 1)], [(0, 1), (1, 16)], [(0, 16)], [(1, 1), (0, 9)]])
    for r in xs:
        assert _rel(whole[r], refs[r]) < TOL[dtype]
        assert _rel(cut[r], refs[r]) < TOL[dtype]
        assert torch.equal(whole[r], cut[r]), "a token's result must not depend on the cut or on the batch"


def _channel_weights(rng, H, heads, kv_heads, dim, vdim, taps, ra, rg):
    gd, hv, hd = kv_heads * dim, heads * vdim, heads * dim
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (
            ("q", "q", (gd, H), 0.3, 0), ("k", "k", (gd, H), 0.3, 0), ("v", "v", (hv, H), 0.3, 0),
            ("q_conv", "q.conv", (gd, taps), 0.6, 0), ("k_conv", "k.conv", (gd, taps), 0.6, 0),
            ("v_conv", "v.conv", (hv, taps), 0.6, 0), ("b", "b", (heads, H), 0.3, 0),
            ("A_log", "A_log", (heads,), 0.7, 0), ("norm", "norm", (vdim,), 0.2, 1),
            ("a1", "a1", (ra, H), 0.3, 0), ("a2", "a2", (hd, ra), 0.6, 0), ("dt_bias", "dt_bias", (hd,), 1.0, 0),
            ("g1", "g1", (rg, H), 0.3, 0), ("g2", "g2", (hv, rg), 0.6, 0), ("o", "o", (H, hv), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(4, 2, 12, 20, 4), (2, 2, 32, 32, 4), (6, 1, 8, 40, 2),
                                                          (1, 1, 64, 128, 1), (3, 3, 24, 6, 7)])
def test_channel_delta_alone_in_portions_and_beside_another_request(dtype, heads, kv_heads, dim, vdim, taps):
    """Also: portions shorter than the convolution's tail (one and two tokens with up to six taps
    behind), so that the tail is shifted, not replaced."""
    rng = np.random.default_rng(vdim)
    ctx = _ctx(dtype)
    H = 40
    wt, w64 = _channel_weights(rng, H, heads, kv_heads, dim, vdim, taps, 5, 7)
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}
    mixer = _make("mixer", "channel_delta", {"hidden_size": H, "heads": heads, "kv_heads": kv_heads, "dim": dim,
                                             "vdim": vdim, "conv": taps, "decay_rank": 5, "gate_rank": 7,
                                             "eps": 1e-5}, wt, ctx)
    xs, refs = {}, {}
    for r, T in enumerate((45, 19)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), R.channel_delta(x64, w64, "", mx, 1e-5)
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 45)], [(1, 19)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 1), (1, 1)], [(0, 2), (1, 1)], [(0, 1), (1, 16)], [(0, 1)], [(0, 17)],
                                         [(0, 2)], [(0, 20), (1, 1)], [(0, 1)]])
    for r in xs:
        assert _rel(whole[r], refs[r]) < TOL[dtype]
        assert _rel(cut[r], refs[r]) < TOL[dtype]
        assert torch.equal(whole[r], cut[r])


def _latent_weights(rng, H, mx):
    heads, dim, rot, vdim, qr, kr = (mx[k] for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"))
    wt, w64 = {}, {}
    for role, name, shape, std, mean in (
            ("dq", "dq", (qr, H), 0.3, 0), ("dq_norm", "dq.norm", (qr,), 0.2, 1),
            ("uq", "uq", (heads * (dim + rot), qr), 0.5, 0), ("dkv", "dkv", (kr + rot, H), 0.3, 0),
            ("dkv_norm", "dkv.norm", (kr,), 0.2, 1), ("uk", "uk", (heads * dim, kr), 0.5, 0),
            ("uv", "uv", (heads * vdim, kr), 0.5, 0), ("sink", "sink", (heads,), 1.0, 1.0),
            ("o", "o", (H, heads * vdim), 0.3, 0)):
        wt[role], w64[name] = _w(rng, shape, std, mean)
    return wt, w64


def _latent_mixer(mx, wt, ctx, H):
    from kv_cache_optimization_for_llm_b200.models.spec import PartSpec
    rope = PartSpec("rope_interleaved", {"dims": mx["rot"]["dims"], "base": mx["rot"]["base"]})
    return _make("mixer", "latent_attention", {
        "hidden_size": H, "heads": mx["heads"], "dim": mx["dim"], "rot_dim": mx["rot_dim"], "vdim": mx["vdim"],
        "q_rank": mx["q_rank"], "kv_rank": mx["kv_rank"], "scale": mx["scale"], "eps": 1e-5, "position": rope}, wt, ctx)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [dict(), dict(heads=9, dim=8, rot_dim=4, vdim=8, q_rank=12, kv_rank=10),
                                   dict(heads=2, dim=32, rot_dim=16, vdim=16, q_rank=24, kv_rank=72, rot_dims=8),
                                   dict(heads=1, dim=16, rot_dim=64, vdim=8, q_rank=8, kv_rank=200, base=77.0),
                                   # sizes that the tensor-core form takes in bfloat16: three tokens of 20 heads to a
                                   # tile, more heads than one tile has rows, a latent between two of its sizes
                                   dict(heads=3, dim=16, rot_dim=16, vdim=8, q_rank=16, kv_rank=32),
                                   dict(heads=20, dim=8, rot_dim=32, vdim=8, q_rank=8, kv_rank=96, rot_dims=12),
                                   dict(heads=70, dim=8, rot_dim=16, vdim=4, q_rank=8, kv_rank=64),
                                   dict(heads=4, dim=8, rot_dim=16, vdim=8, q_rank=8, kv_rank=160)])
def test_latent_attention_alone_in_portions_and_beside_another_request(dtype, shape):
    """Several shapes (more heads than a block takes, a rotary part of which only some dimensions
    turn, latents wider than one pass over the lanes), 70 and 33 tokens on pages of 8 that lie
    scattered; portions end inside pages and on their borders."""
    rng = np.random.default_rng(3)
    ctx = _ctx(dtype)
    H = 40
    mx = tiny.latent(**shape)["mixer"]
    wt, w64 = _latent_weights(rng, H, mx)
    mixer = _latent_mixer(mx, wt, ctx, H)
    xs, refs = {}, {}
    for r, T in enumerate((70, 33)):
        x, x64 = _w(rng, (T, H), 1.0)
        xs[r], refs[r] = x.to(DT[dtype]).cuda(), R.latent_attention(x64, w64, "", mx, 1e-5)
    from kv_cache_optimization_for_llm_b200 import ops
    before = ops.choices["latent_attention_tc"]
    whole = _run_in_steps(mixer, ctx, xs, [[(0, 70)], [(1, 33)]])
    cut = _run_in_steps(mixer, ctx, xs, [[(0, 8), (1, 1)], [(0, 9), (1, 1)], [(0, 2), (1, 30)], [(0, 1), (1, 1)],
                                         [(0, 44)], [(0, 1)], [(0, 1)], [(0, 4)]])
    on_tensor_cores = dtype == "bfloat16" and mx["kv_rank"] % 32 == 0 and (mx["kv_rank"] + mx["rot_dim"]) % 16 == 0
    assert (ops.choices["latent_attention_tc"] > before) == on_tensor_cores
    for r in xs:
        assert _rel(whole[r], refs[r]) < TOL[dtype]
        assert _rel(cut[r], refs[r]) < TOL[dtype]
        assert torch.equal(whole[r], cut[r])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kv_rank", [16, 32])
def test_latent_attention_finds_one_far_key_and_counts_the_sink_once(dtype, kv_rank):
    """300 tokens; the shared key part of token 5 is blown up so that, for late queries, its score
    stands out among hundreds (random keys would hide a lost page or a wrong block table).  The
    plain result changes by a large factor when that key is taken away, and when the sink is;
    the mixer agrees with the plain result with both in place, in portions that cut pages."""
    rng = np.random.default_rng(11)
    ctx = _ctx(dtype)
    H, T = 40, 300
    # a latent of 32 with a rotated part of 16 runs on tensor cores in bfloat16, a latent of 16 does not
    mx = tiny.latent(heads=2, dim=8, rot_dim=8 if kv_rank == 16 else 16, vdim=8, q_rank=12, kv_rank=kv_rank, base=1e6)["mixer"]
    wt, w64 = _latent_weights(rng, H, mx)
    wt["sink"], w64["sink"] = _w(rng, (2,), 0.1, 4.0)
    x, x64 = _w(rng, (T, H), 1.0)
    x[5] *= 16.0           # a power of two: bfloat16 holds the product exactly
    x64[5] *= 16.0
    ref = R.latent_attention(x64, w64, "", mx, 1e-5)
    without_key = R.latent_attention(np.delete(x64, 5, axis=0), w64, "", mx, 1e-5)
    no_sink = dict(w64, sink=np.full(2, -50.0))
    assert np.abs(ref[6:] - without_key[5:]).max() > 0.3 * np.abs(ref).max(), "the far key must matter"
    assert np.abs(ref - R.latent_attention(x64, no_sink, "", mx, 1e-5)).max() > 0.1 * np.abs(ref).max()
    mixer = _latent_mixer(mx, wt, ctx, H)
    xs = {0: x.to(DT[dtype]).cuda()}
    got = _run_in_steps(mixer, ctx, xs, [[(0, 3)], [(0, 5)], [(0, 120)], [(0, 1)], [(0, 127)], [(0, 2)]] + [[(0, 1)]] * 42)
    # scores of this size carry a bfloat16 rounding of a few hundredths into the exponent; a lost key
    # or sink would show as 0.3 and more (asserted above), so 0.12 still tells them apart
    assert _rel(got[0], ref) < (3e-5 if dtype == "float32" else 0.12)


# --------------------------------------------------------------------------- whole models

def _runner(folder, dtype, **kw):
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    args = dict(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=3, max_num_batched_tokens=256, max_model_len=160,
                use_cuda_graphs=False)
    args.update(kw)
    return ModelRunner(folder, EngineConfig(**args))


def _logit_err(got, ref, dtype="float32"):
    """float32: the largest difference over the largest logit.  bfloat16: root mean square of the
    differences over that of the logits: with head sizes of 8 to 20 single tokens are ill-conditioned
    (a head's read-out five times smaller than usual in front of its RMS norm turns 4 % of rounding
    into 30 % at that token; the plain model with rounded projections shows the same tokens), so a
    maximum says little there."""
    if dtype == "float32":
        return np.abs(got - ref).max() / np.abs(ref).max()
    return np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_model_prefill_decoding_portions_batches_and_reuse(dtype):
    """A model with every kind of layer, a repeated run of layers and ranks that config.json leaves
    to the tensors' shapes.  Whole prompts; token by token; portions of 2, 3, 7, ... beside single
    tokens of another request; then requests that end and others that take over their slots and
    pages in a pool that holds two of them at most; 60 decoded tokens in a row."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_rz_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=1)
    # the file on disk names no ranks: they are the shapes of w1, a1 and g1
    import json
    bare = json.loads(json.dumps(cfg))
    for layer in bare["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(bare, f)
    r = _runner(folder, dtype)
    assert len(r.spec.schedule) == 8 and len(r.cache.states) == 5 and r.cache.group_entries == [2, 1]
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (90, 37, 61, 1, 150)]
    refs = [R.forward(cfg, w, s) for s in seqs]
    tol = TOL_MODEL[dtype]
    # whole, then the same token by token: equal beyond rounding (here: bit for bit)
    whole = r.step([StepEntry(0, seqs[1], 0, range(37))]).cpu().numpy()
    assert _logit_err(whole, refs[1], dtype) < tol
    r.release(0)
    single = np.concatenate([r.step([StepEntry(1, [t], i, [0])]).cpu().numpy() for i, t in enumerate(seqs[1])])
    assert _logit_err(single, refs[1], dtype) < tol
    assert np.array_equal(whole, single)
    r.release(1)
    # portions of request 0 beside single tokens of request 2 (after its first 20), a third request of one token
    got2 = [r.step([StepEntry(12, seqs[2][:20], 0, range(20))]).cpu().numpy()]
    pos0, pos2, got0 = 0, 20, []
    for n in (2, 3, 7, 1, 8, 16, 2, 9, 5, 1, 1, 30, 2, 3):
        entries = [StepEntry(10, seqs[0][pos0:pos0 + n], pos0, range(n))]
        if pos2 < len(seqs[2]):
            entries.insert(0 if n % 2 else 1, StepEntry(12, [seqs[2][pos2]], pos2, [0]))
        if n == 7:
            entries.append(StepEntry(13, seqs[3], 0, [0]))
        out = r.step(entries).cpu().numpy()
        i = 0
        for e in entries:
            k = len(e.want)
            if e.request_id == 10:
                got0.append(out[i:i + k])
            elif e.request_id == 12:
                got2.append(out[i:i + k])
                pos2 += 1
            else:
                assert _logit_err(out[i:i + k], refs[3], dtype) < tol
                r.release(13)
            i += k
        pos0 += n
    assert pos0 == 90
    assert _logit_err(np.concatenate(got0), refs[0], dtype) < tol
    assert _logit_err(np.concatenate(got2), refs[2][:pos2], dtype) < tol
    r.check_status()
    # both end; a long request takes over slots and pages that were just used (the pool holds 320 tokens)
    r.release(10)
    r.release(12)
    assert r.manager.check() == ""
    long = [r.step([StepEntry(20, seqs[4][:90], 0, range(90))]).cpu().numpy()]
    for i in range(90, 150):
        long.append(r.step([StepEntry(20, [seqs[4][i]], i, [0])]).cpu().numpy())
    assert _logit_err(np.concatenate(long), refs[4], dtype) < tol
    r.check_status()
    r.release(20)
    assert all(r.manager.free_pages(g) == 40 for g in range(r.manager.num_groups()))


@pytest.mark.parametrize("layers,loop", [
    ([tiny.latent(heads=2, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=8)], None),
    ([tiny.general(heads=1, dim=32, rank=4, ff=24)], {"start": 0, "stop": 1, "times": 3}),
    ([tiny.channel(heads=2, kv_heads=1, dim=16, vdim=16, conv=3), tiny.latent(ff=32)], {"start": 1, "stop": 2, "times": 1}),
    # sizes that are no powers of two, three layers repeated twice, the attention on tensor cores in bfloat16
    ([tiny.general(heads=3, dim=48, rank=10, ff=72), tiny.channel(heads=6, kv_heads=2, dim=40, vdim=24, conv=3, rank=9, gate_rank=11),
      tiny.latent(heads=5, dim=24, rot_dim=16, vdim=40, q_rank=36, kv_rank=96, rot_dims=8, ff=88),
      tiny.general(heads=1, dim=96, rank=3)], {"start": 0, "stop": 3, "times": 2}),
])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_orders_of_layers_and_loops(layers, loop, dtype):
    """One layer alone, a lone layer three times in a row, a loop of one pass, odd sizes: a prompt in
    three portions and four tokens one by one."""
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    folder = tempfile.mkdtemp(prefix="kvb200_rz_")
    cfg = tiny.config(layers, width=40 if len(layers) < 4 else 104, vocab=53, loop=loop, eps=1e-6)
    w = tiny.write_model(folder, cfg, seed=2)
    r = _runner(folder, dtype)
    seq = np.random.default_rng(1).integers(0, 53, 44).tolist()
    ref = R.forward(cfg, w, seq)
    got, pos = [], 0
    for n in (11, 2, 27, 1, 1, 1, 1):
        got.append(r.step([StepEntry(0, seq[pos:pos + n], pos, range(n))]).cpu().numpy())
        pos += n
    assert _logit_err(np.concatenate(got), ref, dtype) < TOL_MODEL[dtype]
    r.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype):
    """Prompts of unequal length through ``LLM.generate``: the scheduler's portions (a token budget of
    24 per step), decode steps replayed from CUDA graphs, the engine one step ahead, five requests in
    three seats.  Every sampled row's logits are compared with the plain model on the final sequences,
    and in float32 the greedy tokens themselves."""
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    from logit_hook import LogitRecorder
    folder = tempfile.mkdtemp(prefix="kvb200_rz_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=4)
    llm = LLM(folder, dtype=dtype, page_size=8, num_pages=48, max_num_seqs=3, max_num_batched_tokens=24,
              max_model_len=128, use_cuda_graphs=True, run_ahead=True)
    rec = LogitRecorder(llm.engine.runner)
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (3, 41, 17, 1, 30)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    assert [len(o) for o in outs] == [12] * 5
    seqs = {i: prompts[i] + outs[i] for i in range(5)}
    plain = {i: R.forward(cfg, w, seqs[i]) for i in seqs}
    n, worst = rec.compare(seqs, lambda i: plain[i], TOL_MODEL[dtype], "greedy generation")
    assert n >= 60 and llm.engine.runner._graphs
    if dtype == "float32":
        for i in seqs:
            for j, tok in enumerate(outs[i]):
                row = plain[i][len(prompts[i]) + j - 1]
                assert row[tok] >= row.max() - 1e-4 * np.abs(row).max(), (i, j)
    assert llm.engine.runner.manager.check() == ""


@pytest.mark.parametrize("dtype,flags", [("float32", ()), ("bfloat16", ()), ("float32", ("--cuda-graphs",))])
def test_replay_through_the_trace_runner(dtype, flags):
    """bin/trace_run on a Rezusun folder: each request whole, then four live requests whose portions
    (down to two tokens) run beside single tokens in a pool that holds exactly them, in four state
    slots; requests that end hand pages and slots to the ones that follow."""
    from trace_driver import TraceRun, ceil64
    folder = tempfile.mkdtemp(prefix="kvb200_rz_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=6)
    rng = np.random.default_rng(2)
    seqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (70, 33, 50, 21)]
    refs = [R.forward(cfg, w, s) for s in seqs]
    tol = TOL_MODEL[dtype]
    tr = TraceRun(folder, dtype, sum(ceil64(len(s)) for s in seqs), ("--page-size", "8") + tuple(flags))
    try:
        for r, s in enumerate(seqs):
            got = tr.step([(f"w{r}", s, range(len(s)))], end=[f"w{r}"])
            assert _logit_err(got, refs[r], dtype) < tol, f"whole request {r}"
        for round_ in range(2):         # the second round runs in slots and pages that the first gave back
            plans = {0: [5, 2, 16, 9, 2, 30] + [1] * 6, 1: [1, 1, 20, 2] + [1] * 9, 2: [33, 2, 3, 2] + [1] * 10,
                     3: [2, 2, 2, 7] + [1] * 8}
            pos = {r: 0 for r in plans}
            step = 0
            while plans:
                entries, expect, ends = [], [], []
                for r in sorted(plans):
                    if step < r:        # they start one step apart
                        continue
                    n = plans[r].pop(0)
                    entries.append((f"m{round_}_{r}", seqs[r][pos[r]:pos[r] + n], range(n)))
                    expect.append(refs[r][pos[r]:pos[r] + n])
                    pos[r] += n
                    if not plans[r]:
                        assert pos[r] == len(seqs[r])
                        ends.append(f"m{round_}_{r}")
                        del plans[r]
                got = tr.step(entries, end=ends)
                assert _logit_err(got, np.concatenate(expect), dtype) < tol, f"round {round_}, mixed step {step}"
                step += 1
    finally:
        tr.close()


def test_command_line_serves_the_design():
    """The engine's command line on a Rezusun folder: requests on standard input in the wire format,
    greedy tokens back as JSON lines; each token is the plain model's best (ties within 1e-4 allowed)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = tempfile.mkdtemp(prefix="kvb200_rz_")
    cfg = tiny.MIXED
    w = tiny.write_model(folder, cfg, seed=8)
    rng = np.random.default_rng(4)
    prompts = {3: rng.integers(0, cfg["vocab"], 9).tolist(), 11: rng.integers(0, cfg["vocab"], 26).tolist()}
    lines = [f"{rid} 6 1 " + " ".join(map(str, toks)) for rid, toks in prompts.items()]
    env = dict(os.environ, IGNORE_EOS="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-m", "kv_cache_optimization_for_llm_b200.cli", folder, "--dtype", "float32",
                        "--page-size", "4", "--num-pages", "64", "--max-num-seqs", "4", "--max-model-len", "64"],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [json.loads(line) for line in p.stdout.splitlines() if line.strip()]
    for rid, prompt in prompts.items():
        toks = [m["tok"] for m in out if m.get("id") == rid and "tok" in m]
        assert len(toks) == 6
        logits = R.forward(cfg, w, prompt + toks)
        for j, tok in enumerate(toks):
            row = logits[len(prompt) + j - 1]
            assert row[tok] >= row.max() - 1e-4 * np.abs(row).max(), (rid, j)
