"""Deletar in the engine against the plain implementation (``plain_deletar``): each mechanism alone, the kernels
alone, whole prompts against decoding and against portions, mixed batches on small pools with pages and state
rows handed on, keys at the windows' edges and at page borders made visible by the weights, the convolution's reach,
borrowed keys read through another window, long decoding, other sizes, greedy generation through ``LLM``.  Every test
builds its own tiny model with random weights."""

import json
import math
import os
import random

import numpy as np
import pytest
import torch

import plain_deletar as plain
import replay_cases as rc

pytestmark = pytest.mark.gpu

VOCAB = 131


# ----------------------------------------------------------------------------- tiny models
def dense(ff=40):
    return dict(kind="dense", ff=ff)


def experts(ff=24, experts=5, top=2, shared=16):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


def banded(factor=4.0, low=1.0, high=3.0, original=40):
    return dict(factor=factor, low=low, high=high, original=original)


def mixer(heads=4, kv_heads=2, dim=8, vdim=8, window=13, dims=4, base=100.0, scale=0.3, softcap=None, scaling=None, conv=None, kv_from=None):
    rot = dict(dims=dims, base=base)
    if scaling is not None:
        rot["scaling"] = scaling
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rot)
    if window is not None:
        m["mask"] = dict(size=window)
    if softcap is not None:
        m["softcap"] = softcap
    if conv is not None:
        m["conv"] = conv
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def conv_layer(mlp=dense(), conv=3, vdim=12, **kw):
    return dict(type="attention", mixer=mixer(conv=conv, vdim=vdim, **kw), mlp=mlp)


def keys_as_values_layer(mlp=dense(), softcap=9.0, **kw):
    return dict(type="attention_2", mixer=mixer(softcap=softcap, **kw), mlp=mlp)


def sink_layer(mlp=dense(), softcap=7.0, vdim=6, heads=6, kv_heads=2, **kw):
    return dict(type="attention_3", mixer=mixer(softcap=softcap, vdim=vdim, heads=heads, kv_heads=kv_heads, **kw), mlp=mlp)


def model_config(layers, width=48, vocab=VOCAB, eps=1e-5, scale=5.0, softcap=11.0):
    cfg = dict(architecture="Deletar", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=scale), layers=layers)
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


# all three mixers, a layer that borrows keys through a wider window than their owner's, experts and a dense feed-forward,
# a layer without a feed-forward; the sink layers' heads are of a size the tensor-core kernel takes (16), the others' not
HYBRID = model_config([
    keys_as_values_layer(mlp=dense()),
    sink_layer(dim=16, vdim=16, dims=8, window=9, scaling=banded(), mlp=experts()),
    conv_layer(conv=4, mlp=experts(ff=16, experts=3, top=3, shared=0)),
    keys_as_values_layer(heads=3, kv_heads=3, dim=12, vdim=12, dims=12, window=21, mlp=None),
    sink_layer(dim=16, vdim=16, dims=8, window=17, scaling=banded(), kv_from=1, mlp=experts(ff=8, experts=7, top=1)),
])


def make_folder(tmp_path, cfg, seed=3, edits=None, name="m", std=0.08) -> str:
    """A model folder with bfloat16-representable random weights; ``edits``: tensor name -> function
    that changes the float32 tensor in place."""
    from safetensors.torch import save_file

    from tandem_b200.config.deletar_config import DeletarConfig
    from tandem_b200.models.deletar import random_weights

    typed = DeletarConfig.from_dict(json.loads(json.dumps(cfg)))
    tensors = {}
    for tensor_name, t in random_weights(typed, seed, "cpu", torch.float32, std=std):
        if edits and tensor_name in edits:
            edits[tensor_name](t)
        tensors[tensor_name] = (t if t.dtype == torch.int32 else t.to(torch.bfloat16)).contiguous()
    folder = os.path.join(str(tmp_path), name)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


def tokens(seed, n, vocab=VOCAB):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_steps(folder, dtype, steps, page_size=4, pool_tokens=None, max_requests=4, log=None):
    """The steps through the engine's step function; request id -> [positions, vocab] float64."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.kernels import ops

    decoder, _ = load_model(folder, dtype, "cuda:0")
    need = pool_tokens if pool_tokens is not None else rc.tokens_needed(steps, round_to=max(16, page_size))
    ex = build_executor(decoder, page_size=page_size, num_pages=-(-need // page_size), max_requests=max_requests)
    if log is not None:
        log.append(rc.PageLog(ex.manager))
    out = {}
    for st in steps:
        logits = ex.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]], end=st["end"])
        if logits.shape[0]:
            out[st["step"]] = logits.cpu().double().numpy()
        ex.manager.check()
    ops.check_status(ex.device)
    assert ex.manager.all_free()
    return {rid: torch.from_numpy(np.stack(rows)) for rid, rows in rc.collect(steps, out).items()}


def per_position(got, ref):
    """Root mean square over the vocabulary of the difference (mean taken off), over that of the reference's logits."""
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / r.pow(2).mean().sqrt()


def distance(got, ref):
    return float(per_position(got, ref).max())


LIMIT = {"float32": 3e-5, "bfloat16": 5e-2}


def agrees(got, ref, dtype) -> bool:
    return distance(got, ref) < LIMIT[dtype]


def reference(folder, requests):
    cfg, w = plain.read_folder(folder)
    return {rid: plain.forward(cfg, w, t)[0] for rid, t in requests.items()}


# ----------------------------------------------------------------------------- each mechanism alone
ALONE = {
    "convolved": model_config([conv_layer(mlp=None)]),
    "convolved_one_tap": model_config([conv_layer(conv=1, mlp=None)]),
    "convolved_two_taps": model_config([conv_layer(conv=2, mlp=None)]),
    "convolved_nine_taps_capped": model_config([conv_layer(conv=9, softcap=3.0, heads=2, kv_heads=1, mlp=None)]),
    "convolved_tensor_cores": model_config([conv_layer(conv=4, heads=4, kv_heads=1, dim=32, vdim=16, dims=32, mlp=None)]),
    "keys_as_values": model_config([keys_as_values_layer(mlp=None)]),
    "keys_as_values_one_head": model_config([keys_as_values_layer(heads=1, kv_heads=1, dim=20, vdim=20, dims=2, mlp=None)]),
    "keys_as_values_banded_uncapped": model_config([keys_as_values_layer(softcap=None, dims=8, scaling=banded(), mlp=None)]),
    "keys_as_values_tensor_cores": model_config([keys_as_values_layer(heads=8, kv_heads=2, dim=16, vdim=16, dims=16, mlp=None)]),
    "sink": model_config([sink_layer(mlp=None)]),
    "sink_banded_all_pairs": model_config([sink_layer(dims=8, scaling=banded(factor=8.0, low=0.5, high=0.6, original=4), mlp=None)]),
    "sink_banded_no_pair": model_config([sink_layer(dims=8, base=2.0, scaling=banded(factor=8.0, low=1.0, high=2.0, original=4000), mlp=None)]),
    "sink_as_many_key_heads": model_config([sink_layer(heads=3, kv_heads=3, mlp=None)]),
    "sink_window_of_one": model_config([sink_layer(window=1, mlp=None)]),
    "no_window": model_config([sink_layer(window=None, mlp=None), conv_layer(window=None, mlp=None)]),
    "borrowed_keys": model_config([sink_layer(mlp=None), sink_layer(kv_from=0, window=13, mlp=None)]),
    "borrowed_through_a_wider_window": model_config([sink_layer(window=5, mlp=None), keys_as_values_layer(mlp=None),
                                                     sink_layer(kv_from=0, window=19, mlp=None), sink_layer(kv_from=0, window=3, mlp=None)]),
    "borrowed_without_a_window": model_config([sink_layer(window=5, mlp=None), sink_layer(kv_from=0, window=None, mlp=None)]),
    "dense": model_config([keys_as_values_layer(mlp=dense(ff=56))]),
    "experts": model_config([keys_as_values_layer(mlp=experts())]),
    "experts_without_a_shared_one": model_config([conv_layer(mlp=experts(shared=0))]),
    "one_expert_of_one": model_config([sink_layer(mlp=experts(ff=9, experts=1, top=1, shared=5))]),
    "all_experts": model_config([sink_layer(mlp=experts(ff=16, experts=4, top=4))]),
    "no_softcap_no_scale": model_config([keys_as_values_layer()], softcap=None, scale=1.0),
    "odd_width": model_config([conv_layer(mlp=experts(ff=10, experts=3, top=2, shared=7)), sink_layer()], width=30, vocab=77),
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = ALONE[name]
    folder = make_folder(tmp_path, cfg)
    requests = {"a": tokens(1, 45, cfg["vocab"]), "b": tokens(2, 1, cfg["vocab"])}
    ref = reference(folder, requests)
    got = run_steps(folder, dtype, rc.whole(requests))
    for rid in requests:
        assert agrees(got[rid], ref[rid], dtype), (name, rid, distance(got[rid], ref[rid]))


def test_the_stream_after_every_layer_is_the_plain_one(tmp_path):
    """What stands in the stream once a layer's last output has been normed and added, in float32."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry

    folder = make_folder(tmp_path, HYBRID)
    toks = tokens(5, 30)
    cfg, w = plain.read_folder(folder)
    _, layers = plain.forward(cfg, w, toks)
    decoder, _ = load_model(folder, "float32", "cuda:0")
    ex = build_executor(decoder, page_size=8, num_pages=8, max_requests=2)
    seen = []
    for layer in decoder.layers:
        inner = layer.block.forward

        def spy(l, x, residual, ctx, inner=inner):
            out = inner(l, x, residual, ctx)
            y = out.y.double()
            normed = y / torch.sqrt((y * y).mean(-1, keepdim=True) + out.eps) * out.weight.double()
            seen.append((residual.double() + normed).cpu())
            return out

        layer.block.forward = spy
    ex.step([StepEntry("a", toks, [0])], end=["a"])
    assert len(seen) == len(layers) == 5
    for i, (g, r) in enumerate(zip(seen, layers)):
        assert (g - r).abs().max() < 1e-5 * max(1.0, float(r.abs().max())), i


# ----------------------------------------------------------------------------- the kernels alone
class Batch:
    """The device arrays of a step that the kernels read."""

    def __init__(self, starts, lens, slots):
        seq, pos, cu = [], [], [0]
        for b, (s, n) in enumerate(zip(starts, lens)):
            seq += [b] * n
            pos += list(range(s, s + n))
            cu.append(cu[-1] + n)
        as_int = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
        self.seq_of_token, self.positions, self.cu_seqlens = as_int(seq), as_int(pos), as_int(cu)
        self.seq_starts, self.state_slots, self.num_seqs = as_int(starts), as_int(slots), len(lens)


class Cache:
    """A paged cache of one request per row of the block table, pages handed out in a scrambled order."""

    def __init__(self, nkv, dk, dv, page_size, lens, dtype):
        from tandem_b200.parts.base import KVView

        pages = [-(-n // page_size) for n in lens]
        order = list(range(sum(pages) + 3))
        random.Random(7).shuffle(order)
        self.table = torch.full((len(lens), max(pages)), -1, dtype=torch.int32)
        at = 0
        for b, n in enumerate(pages):
            self.table[b, :n] = torch.tensor(order[at: at + n], dtype=torch.int32)
            at += n
        self.page_size = page_size
        self.k = torch.zeros(len(order), nkv, page_size, dk, dtype=dtype).cuda()
        self.v = torch.zeros(len(order), nkv, page_size, dv, dtype=dtype).cuda()
        self.view = lambda slots: KVView(self.k, self.v, self.table.cuda(), slots, page_size, writable=True)

    def slots(self, starts, lens):
        out = []
        for b, (s, n) in enumerate(zip(starts, lens)):
            out += [int(self.table[b, p // self.page_size]) * self.page_size + p % self.page_size for p in range(s, s + n)]
        return torch.tensor(out, dtype=torch.int32).cuda()

    def rows(self, which, b, n):
        """The first n rows of request b as [n, heads, dim], through the package's own map of a tile."""
        from tandem_b200.cache.layout import to_logical

        t = to_logical(self.k if which == "k" else self.v)
        pages = [t[int(p)] for p in self.table[b] if p >= 0]  # each [heads, page_size, dim]
        return torch.cat(pages, dim=1).transpose(0, 1)[:n].double().cpu()


@pytest.mark.parametrize("norm,taps,rot,values_from_keys,has_bias", [("none", 3, 4, False, False), ("whole", 0, 8, True, True), ("head", 0, 2, False, False),
                                                                       ("unit", 2, 0, False, True), ("head", 5, 6, False, False)])
def test_the_prepare_kernel_against_the_plain_pieces(norm, taps, rot, values_from_keys, has_bias):
    """Bias, convolution over steps whose borders fall inside its reach (with stale numbers in other requests' state rows),
    the three norms, the partial rotation and the cache write, against float64."""
    from tandem_b200.kernels import post_norm, sink_attention as sa

    nh, nkv, dk = 4, 2, 8
    dv = dk if values_from_keys else 12
    g = torch.Generator().manual_seed(taps * 10 + rot)
    lens_total = [23, 9]
    q_cols, k_cols, v_cols = nh * dk, nkv * dk, 0 if values_from_keys else nkv * dv
    cols = q_cols + k_cols + v_cols
    raw = [torch.randn(n, cols + 3, generator=g) for n in lens_total]  # three more columns stand for a gate's
    bias = torch.randn(cols, generator=g) if has_bias else None
    tap_w = torch.randn(cols, taps, generator=g) * 0.5 if taps else None
    q_w = torch.rand(dk if norm == "head" else q_cols, generator=g) + 0.5 if norm in ("head", "whole") else None
    k_w = torch.rand(dk if norm == "head" else k_cols, generator=g) + 0.5 if norm in ("head", "whole") else None
    freq = plain.frequencies(rot, 50.0) if rot else None
    eps = 1e-3
    want = []
    for x in raw:
        u = x[:, :cols].double() + (bias.double() if has_bias else 0.0)
        if taps:
            u = plain.causal_convolution(u, tap_w.double())
        q, k = u[:, :q_cols], u[:, q_cols: q_cols + k_cols]
        v = k.clone() if values_from_keys else u[:, q_cols + k_cols:]
        if norm == "whole":
            q, k = plain.norm_plain(q, q_w.double(), eps), plain.norm_plain(k, k_w.double(), eps)
        q, k = q.reshape(-1, nh, dk), k.reshape(-1, nkv, dk)
        if norm == "head":
            q, k = plain.norm_plain(q, q_w.double(), eps), plain.norm_plain(k, k_w.double(), eps)
        if norm == "unit":
            q, k = plain.rms(q, eps), plain.rms(k, eps)
        if rot:
            q, k = plain.rotate(q, freq, rot), plain.rotate(k, freq, rot)
        want.append((q, k, v.reshape(-1, nkv, dv)))
    cache = Cache(nkv, dk, dv, 4, lens_total, torch.float32)
    state = torch.full((5, max(taps - 1, 1), cols), 7.0).cuda()
    state[3].zero_()
    state[1].zero_()
    at, got_q = [0, 0], [[], []]
    for cut in ((1, 2), (2, 1), (5, 2), (1, 1), (14, 3)):
        b = Batch(at, list(cut), [3, 1])
        proj = torch.cat([raw[i][at[i]: at[i] + cut[i]] for i in range(2)]).cuda().contiguous()
        q = sa.prepare_rows(proj, cache.view(cache.slots(at, cut)), b, nh, nkv, dk, dv, bias=None if bias is None else bias.cuda(),
                            taps=None if tap_w is None else tap_w.t().contiguous().cuda(), state=state if taps > 1 else None, qk_norm=norm,
                            q_weight=None if q_w is None else q_w.cuda(), k_weight=None if k_w is None else k_w.cuda(), eps=eps,
                            freq=None if freq is None else torch.tensor(freq, dtype=torch.float32).cuda(), values_from_keys=values_from_keys)
        if taps > 1:
            post_norm.short_conv_state(proj, state, b, taps, width=cols)
        o = 0
        for i in range(2):
            got_q[i].append(q[o: o + cut[i]].cpu())
            o += cut[i]
        at = [at[i] + cut[i] for i in range(2)]
    for i in range(2):
        n = lens_total[i]
        assert (torch.cat(got_q[i]).double().view(n, nh, dk) - want[i][0]).abs().max() < 2e-5
        assert (cache.rows("k", i, n) - want[i][1]).abs().max() < 2e-5
        assert (cache.rows("v", i, n) - want[i][2]).abs().max() < 2e-5
    assert torch.equal(state[[0, 2, 4]], torch.full_like(state[[0, 2, 4]], 7.0))  # nobody else's rows were touched


def test_the_rotation_far_out_with_slowed_frequencies():
    """Position 3,001 of a request, frequencies slowed between two wavelengths: the float32 angles against float64."""
    from tandem_b200.config.plan import RotaryBandSpec, rotary_band_table
    from tandem_b200.kernels import sink_attention as sa

    nh, nkv, dk, rot = 2, 1, 16, 12
    scaling = dict(factor=6.0, low=1.0, high=4.0, original=64)
    freq = plain.frequencies(rot, 300.0, scaling)
    assert freq == rotary_band_table(rot, 300.0, RotaryBandSpec(6.0, 1.0, 4.0, 64))
    plain_freq = plain.frequencies(rot, 300.0)
    assert freq[0] == plain_freq[0] and abs(freq[-1] - plain_freq[-1] / 6.0) < 1e-15 and any(
        b / 6.0 < a < b for a, b in zip(freq, plain_freq))  # kept, slowed, and between
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, (nh + 2 * nkv) * dk, generator=g)
    start = 3000
    cache = Cache(nkv, dk, dk, 16, [start + 2], torch.float32)
    b = Batch([start], [2], [0])
    q = sa.prepare_rows(x.cuda(), cache.view(cache.slots([start], [2])), b, nh, nkv, dk, dk,
                        freq=torch.tensor(freq, dtype=torch.float32).cuda())
    padded = torch.zeros(start + 2, nh, dk, dtype=torch.float64)
    padded[start:] = x[:, :nh * dk].double().view(2, nh, dk)
    want = plain.rotate(padded, freq, rot)[start:]
    assert (q.cpu().double().view(2, nh, dk) - want).abs().max() < 3001 * 2.0 ** -23  # the rounding of an angle of 3,001, not more
    assert (q.cpu().double().view(2, nh, dk) - x[:, :nh * dk].double().view(2, nh, dk)).abs().max() > 0.1


@pytest.mark.parametrize("H,y_dtype,out_dtype", [(48, "float32", "float32"), (1280, "bfloat16", "bfloat16"), (30, "float32", "bfloat16"),
                                                 (4100, "float32", "float32")])
def test_norm_add_norm(H, y_dtype, out_dtype):
    """A sublayer's output normed and added, the stream normed for the next sublayer: one launch against float64, on all
    rows and on gathered rows, and the add alone."""
    from tandem_b200.kernels import ops

    g = torch.Generator().manual_seed(H)
    yt, ot = getattr(torch, y_dtype), getattr(torch, out_dtype)
    T = 37
    y = (torch.randn(T, H, generator=g) * 3).to(yt)
    x = torch.randn(T, H, generator=g)
    wy, w = torch.rand(H, generator=g) + 0.5, torch.rand(H, generator=g) + 0.5
    stream = x.double() + plain.norm_plain(y.double(), wy.double(), 1e-3)
    want = plain.norm_plain(stream, w.double(), 1e-5)
    res = x.clone().cuda()
    out = ops.norm_add_norm(y.cuda(), wy.cuda(), 1e-3, res, w.cuda(), 1e-5, ot)
    tol = 2.0 ** -7 if out_dtype == "bfloat16" else 1e-5
    assert (res.cpu().double() - stream).abs().max() < 1e-5
    assert (out.cpu().double() - want).abs().max() < tol * float(want.abs().max())
    rows = torch.tensor([5, 0, 36], dtype=torch.int32)
    res2 = x.clone().cuda()
    out2 = ops.norm_add_norm(y.cuda(), wy.cuda(), 1e-3, res2, w.cuda(), 1e-5, ot, rows=rows.cuda())
    assert torch.equal(out2.cpu(), out.cpu()[rows.long()])
    untouched = [i for i in range(T) if i not in (5, 0, 36)]
    assert torch.equal(res2.cpu()[untouched], x[untouched])
    res3 = x.clone().cuda()
    assert ops.norm_add_norm(y.cuda(), wy.cuda(), 1e-3, res3, None, 1e-5, ot) is None
    assert torch.equal(res3, res)


@pytest.mark.parametrize("T,top,real,ff,width,dtype", [(7, 2, 6, 24, 64, "float32"), (7, 1, 2, 40, 48, "bfloat16"), (90, 3, 5, 16, 96, "bfloat16"),
                                                       (600, 2, 4, 64, 128, "bfloat16"), (90, 4, 4, 10, 30, "float32")])
def test_experts_named_by_a_table_with_the_squared_relu(T, top, real, ff, width, dtype):
    """Routing by token id and experts down(relu(up x)^2) on the three paths (a warp per output, sorted tiles, the grouped
    product), against float64."""
    from tandem_b200.kernels import moe

    g = torch.Generator().manual_seed(T + top)
    dt = getattr(torch, dtype)
    vocab = 50
    table = torch.rand(vocab, real, generator=g).argsort(dim=1)[:, :top].to(torch.int32).contiguous()
    toks = torch.randint(0, vocab, (T,), generator=g, dtype=torch.int32)
    x = torch.randn(T, width, generator=g).to(dt)
    up = (torch.randn(real, ff, width, generator=g) * 0.2).to(dt)
    down = (torch.randn(real, width, ff, generator=g) * 0.2).to(dt)
    ids, weights = moe.route_table(toks.cuda(), table.cuda(), real)
    assert torch.equal(ids.cpu(), table[toks.long()]) and torch.equal(weights.cpu(), torch.full((T, top), 1.0 / top))
    got = moe.experts(x.cuda(), up.cuda(), down.cuda(), ids, weights, gated=False, activation="relu2").cpu().double()
    want = torch.zeros(T, width, dtype=torch.float64)
    for t in range(T):
        for e in table[int(toks[t])].tolist():
            a = plain.relu_squared(x[t].double() @ up[e].double().T)
            if dtype == "bfloat16":
                a = a.to(torch.bfloat16).double()  # the activations are product operands
            want[t] += a @ down[e].double().T / top
    assert (got - want).abs().max() < (2e-2 if dtype == "bfloat16" else 1e-4) * float(want.abs().max())


@pytest.mark.parametrize("dtype,dk,dv,tokens_per_request", [("float32", 8, 12, (5, 1)), ("bfloat16", 16, 16, (40, 3)), ("bfloat16", 16, 32, (1, 1)),
                                                            ("bfloat16", 12, 8, (1, 1))])
def test_the_heads_gate_in_the_attention_kernels(dtype, dk, dv, tokens_per_request):
    """Every head's output times the sigmoid of its number, inside each of the three attention kernels: the gated call
    against the plain call times the gate."""
    from tandem_b200.kernels import sink_attention as sa

    nh, nkv, page = 4, 2, 4
    dt = getattr(torch, dtype)
    g = torch.Generator().manual_seed(dk)
    before = [30, 9]
    total = [a + b for a, b in zip(before, tokens_per_request)]
    cache = Cache(nkv, dk, dv, page, total, dt)
    cache.k.copy_(torch.randn(cache.k.shape, generator=g).to(dt))
    cache.v.copy_(torch.randn(cache.v.shape, generator=g).to(dt))
    b = Batch(before, list(tokens_per_request), [0, 1])
    T = sum(tokens_per_request)
    q = torch.randn(T, nh * dk, generator=g).cuda()
    gate_rows = torch.randn(T, nh + 5, generator=g).cuda()
    gate = gate_rows[:, 2: 2 + nh]  # rows of a wider tensor
    kv = cache.view(cache.slots(before, tokens_per_request))
    sink = torch.zeros(nh).cuda()
    args = (nh, nkv, dk, dv, 11, 0, 0.3, 5.0, None, sink)
    calls = [lambda **kw: sa.attend(q, kv, b, *args, **kw)]
    if max(tokens_per_request) == 1 and sa.split_applies(dt, dk, dv, nh // nkv, nh * dk):
        calls.append(lambda **kw: sa.attend_split(q, kv, b, *args, **kw))
    if dtype == "bfloat16" and sa.tiles_apply(dt, dk, dv, nh // nkv, nh * dk):
        tiles = torch.tensor(sa.plan_tiles(before, list(tokens_per_request), nh // nkv), dtype=torch.int32).cuda()
        calls.append(lambda **kw: sa.attend_tiles(q, kv, tiles, *args, **kw))
    assert len(calls) >= (1 if dtype == "float32" else 2)
    first = None
    for call in calls:
        plain_out = call().float().view(T, nh, dv)
        gated = call(gate=gate).float().view(T, nh, dv)
        want = plain_out * torch.sigmoid(gate)[:, :, None]
        assert (gated - want).abs().max() < (2.0 ** -7 if dtype == "bfloat16" else 1e-6) * float(want.abs().max())
        first = plain_out if first is None else first
        assert (plain_out - first).abs().max() < (3e-2 if dtype == "bfloat16" else 1e-6) * float(first.abs().max())


# ----------------------------------------------------------------------------- schedules
@pytest.fixture(scope="module")
def hybrid(tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("hybrid"), HYBRID)
    requests = {"a": tokens(11, 97), "b": tokens(12, 33), "c": tokens(13, 64), "d": tokens(14, 2), "e": tokens(15, 50), "f": tokens(16, 1)}
    return folder, requests, reference(folder, requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [1, 4, 16])
def test_prefill_against_token_by_token_decoding(hybrid, dtype, page_size):
    folder, requests, ref = hybrid
    whole = run_steps(folder, dtype, rc.whole(requests), page_size)
    tail = run_steps(folder, dtype, rc.tail_one_by_one(requests, tail=40), page_size)
    for rid in requests:
        assert agrees(whole[rid], ref[rid], dtype), rid
        assert agrees(tail[rid], ref[rid], dtype), rid
        if dtype == "float32":  # every kernel sums in an order that does not depend on the cut
            assert torch.equal(whole[rid], tail[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(hybrid, dtype):
    """Portions shorter than the convolution's reach (four taps) and than the windows."""
    folder, requests, ref = hybrid
    whole = run_steps(folder, dtype, rc.whole(requests), 4) if dtype == "float32" else None
    for sizes in ((2,), (3, 2, 7, 2, 19, 2), (16, 2, 5)):
        got = run_steps(folder, dtype, rc.changing_portions(requests, sizes=sizes), 4)
        for rid in requests:
            assert agrees(got[rid], ref[rid], dtype), (sizes, rid)
            if whole is not None:
                assert torch.equal(got[rid], whole[rid]), (sizes, rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_on_a_small_pool(hybrid, dtype):
    """Up to three live requests, portions beside single tokens; the pool holds only what is live, the state
    tensors have three rows: pages and rows go to new holders while other requests are being read."""
    folder, requests, ref = hybrid
    steps = rc.mixed(requests, live=3, portion=9, decode_after=0.5)
    log = []
    got = run_steps(folder, dtype, steps, page_size=4, pool_tokens=rc.tokens_needed(steps, round_to=4), max_requests=3, log=log)
    assert log[0].pages_reused > 0 and log[0].reused_beside_live > 0
    alone = run_steps(folder, dtype, rc.whole(requests), 4)
    for rid in requests:
        assert agrees(got[rid], ref[rid], dtype), rid
        if dtype == "float32":
            assert torch.equal(got[rid], alone[rid]), rid
        else:
            assert distance(got[rid], alone[rid]) < LIMIT[dtype], rid


def test_a_state_row_that_is_used_again_starts_from_zero(tmp_path):
    """One row for all: the second request finds the first one's projected rows there."""
    folder = make_folder(tmp_path, model_config([conv_layer(conv=4), conv_layer(conv=2, mlp=None)]))
    requests = {"first": tokens(1, 40), "second": tokens(2, 25), "third": tokens(3, 2), "fourth": tokens(4, 1)}
    ref = reference(folder, requests)
    got = run_steps(folder, "float32", rc.tail_one_by_one(requests, tail=5), page_size=8, max_requests=1)
    for rid in requests:
        assert distance(got[rid], ref[rid]) < LIMIT["float32"], rid


def test_long_decoding(tmp_path):
    """Three hundred tokens one by one: the windows pass over decoded tokens many times, pages behind them go back to
    the pool (which holds less than the request) and the convolutions' inputs are carried all the way."""
    folder = make_folder(tmp_path, HYBRID)
    requests = {"a": tokens(21, 330)}
    ref = reference(folder, requests)
    steps = rc.tail_one_by_one(requests, tail=300)
    for dtype in ("float32", "bfloat16"):
        got = run_steps(folder, dtype, steps, page_size=8)
        assert agrees(got["a"], ref["a"], dtype), dtype


def test_pages_behind_the_window_go_back_to_the_pool(tmp_path):
    """A request of 200 tokens in a pool of 64: every layer's window (the widest reader's, where keys are borrowed) fits."""
    folder = make_folder(tmp_path, HYBRID)
    requests = {"a": tokens(22, 200), "b": tokens(23, 90)}
    ref = reference(folder, requests)
    steps = rc.changing_portions(requests, sizes=(5, 2, 9))
    got = run_steps(folder, "float32", steps, page_size=4, pool_tokens=64, max_requests=1)
    for rid in requests:
        assert distance(got[rid], ref[rid]) < LIMIT["float32"], rid


# ----------------------------------------------------------------------------- faults made visible
def zero(t):
    t.zero_()


def quiet(t):
    t.mul_(0.02)


def newest_tap_only(t):
    t.zero_()
    t[:, -1] = 1.0


@pytest.mark.parametrize("kind", ["attention", "attention_2", "attention_3", "borrowed"])
@pytest.mark.parametrize("window,far,page_size", [(40, 13, 16), (33, 31, 16), (64, 16, 8), (7, 300, 4)])
def test_one_loud_key_just_inside_and_just_outside_the_window(tmp_path, kind, window, far, page_size):
    """One token's key and the last tokens' queries are made loud along a number that the rotation leaves alone, so that
    a query's result is that key's value for as long as the key is inside the window, and something else from the next
    position on: the token window - 1 places behind the key sees it, the one after does not.  Prompt, portions (with
    borders at the edge) and single tokens; the key at a page's last and first row and far from both."""
    H, G, d, vocab, W = 4, 2, 8, 60, 48
    key_token, query_token = 59, 58
    m = dict(heads=H, kv_heads=G, dim=d, dims=4, base=100.0, scale=1.0, window=window)
    if kind == "attention":
        layers = [conv_layer(mlp=None, conv=3, vdim=d, **m)]
    elif kind == "attention_2":
        layers = [keys_as_values_layer(mlp=None, softcap=50.0, **m)]
    elif kind == "attention_3":
        layers = [sink_layer(mlp=None, softcap=50.0, vdim=d, **m)]
    else:  # the loud key is layer 0's, read by layer 1 through its own, wider window
        m1 = dict(m, window=max(2, window // 3))
        layers = [sink_layer(mlp=None, softcap=50.0, vdim=d, **m1), sink_layer(mlp=None, softcap=50.0, vdim=d, kv_from=0, **m)]
    cfg = model_config(layers, vocab=vocab, width=W)
    folder = make_folder(tmp_path, cfg)
    _, w = plain.read_folder(folder)
    n = far + window + 6
    toks = [t if t not in (key_token, query_token) else 0 for t in tokens(5, n, vocab)]
    toks[far] = key_token
    for i in range(far + window - 3, n):
        toks[i] = query_token
    reader = len(layers) - 1  # the layer whose queries are loud

    def normed_embedding(token, norm_name):
        return plain.norm_one_plus(w["embed"][token].double() * cfg["embedding"]["scale"], w[norm_name].double(), cfg["norm"]["eps"])

    h_key = normed_embedding(key_token, "l0.norm1")
    h_query = normed_embedding(query_token, "l0.norm1") if reader == 0 else None
    loud = d - 1  # the last number of a head: not rotated

    def loud_key(t):
        quiet(t)
        for head in range(G):
            t[head * d + loud] += (8.0 * h_key / (h_key @ h_key)).float()

    def loud_query(t):
        quiet(t)
        if h_query is not None:
            for head in range(H):
                t[head * d + loud] += (8.0 * h_query / (h_query @ h_query)).float()

    edits = {"l0.mix.k": loud_key, f"l{reader}.mix.q": loud_query}
    for name in ("q", "k", "v"):
        edits[f"l0.mix.{name}.conv"] = newest_tap_only
    if reader == 1:  # layer 1's input is not the embedding alone: a bias in its q norm weight makes every query loud along the number
        def loud_everywhere(t):
            t.fill_(0.05)
            t[loud] = 3.0

        edits["l1.mix.q.norm"] = loud_everywhere
    folder = make_folder(tmp_path, cfg, edits=edits, name="loud")
    requests = {"a": toks}
    ref = reference(folder, requests)
    hidden = list(toks)
    hidden[far] = 0
    without = reference(folder, {"a": hidden})["a"]
    inside, outside = far + window - 1, far + window
    each = per_position(without, ref["a"])
    assert float(each[inside]) > 0.03, "the key matters to the last position that sees it"
    if reader == 0:
        assert float(each[outside:].max()) < 1e-9, "and to none behind it"
    cut = far + window - 2
    schedules = [rc.whole(requests), rc.tail_one_by_one(requests, n - cut), rc.changing_portions(requests, (cut, 2, 2, 3)),
                 rc.changing_portions(requests, (cut + 1, 2, 3)), rc.changing_portions(requests, (5, 2))]
    for dtype in ("float32", "bfloat16"):
        for steps in schedules:
            got = run_steps(folder, dtype, steps, page_size=page_size)
            # loud scores carry the rounding of bfloat16 keys into the weights: twice the usual distance there
            assert distance(got["a"], ref["a"]) < LIMIT[dtype] * (2.0 if dtype == "bfloat16" else 1.0), (dtype, len(steps))
            seen, unseen = per_position(got["a"], ref["a"])[inside], per_position(got["a"], without)[inside]
            assert float(seen) < 0.3 * float(unseen), (dtype, len(steps))  # the engine's last look at the key is a look at it


def test_the_convolutions_oldest_tap_and_no_further(tmp_path):
    """All weight on the oldest tap: a token's query, key and value are those of the token taps - 1 places earlier, in
    prompts, across portion borders and token by token; a model with one tap more or less is another model."""
    def oldest_only(t):
        t.zero_()
        t[:, 0] = 1.0

    results = {}
    for taps in (3, 4, 5):
        cfg = model_config([conv_layer(conv=taps, mlp=None, window=9)])
        edits = {f"l0.mix.{n}.conv": oldest_only for n in ("q", "k", "v")}
        folder = make_folder(tmp_path, cfg, edits=edits, name=f"taps{taps}")
        requests = {"a": tokens(8, 41), "b": tokens(9, 3)}
        ref = reference(folder, requests)
        results[taps] = ref["a"]
        for steps in (rc.whole(requests), rc.tail_one_by_one(requests, 30), rc.changing_portions(requests, (2,)),
                      rc.changing_portions(requests, (3, 5, 2))):
            got = run_steps(folder, "float32", steps, page_size=4)
            for rid in requests:
                assert distance(got[rid], ref[rid]) < LIMIT["float32"], (taps, rid)
    assert distance(results[3], results[4]) > 0.05 and distance(results[5], results[4]) > 0.05


def test_the_sink_and_the_cap_change_the_result(tmp_path):
    """The oracle itself tells the sink, the cap and the gate apart (a kernel that left one out would not pass the tests
    above): with loud keys the one in the denominator matters."""
    cfg = model_config([sink_layer(mlp=None, softcap=2.0, scale=2.0)])
    folder = make_folder(tmp_path, cfg, std=0.3)
    requests = {"a": tokens(3, 30)}
    ref = reference(folder, requests)["a"]
    config, w = plain.read_folder(folder)
    uncapped = json.loads(json.dumps(config))
    uncapped["layers"][0]["mixer"]["softcap"] = 200.0
    assert distance(plain.forward(uncapped, w, requests["a"])[0], ref) > 0.01
    as_keys = json.loads(json.dumps(config))
    as_keys["layers"][0]["type"] = "attention"  # no sink, no norm, no gate
    assert distance(plain.forward(as_keys, {**w, "l0.mix.q.conv": torch.ones(1, 1), "l0.mix.k.conv": torch.ones(1, 1), "l0.mix.v.conv": torch.ones(1, 1)},
                                  requests["a"])[0], ref) > 0.01
    for dtype in ("float32", "bfloat16"):
        got = run_steps(folder, dtype, rc.tail_one_by_one(requests, 10))
        assert distance(got["a"], ref) < LIMIT[dtype]


# ----------------------------------------------------------------------------- other sizes
def random_mixer(rng, index, earlier):
    kind = rng.choice(["attention", "attention_2", "attention_3", "attention_3"])
    kv_heads = rng.choice([1, 2, 3])
    heads = kv_heads * rng.choice([1, 2, 4])
    dim = rng.choice([4, 8, 12, 16, 32])
    vdim = dim if kind == "attention_2" else rng.choice([4, 8, 16, 20])
    dims = rng.choice([d for d in (2, 4, 8, 16, 32) if d <= dim])
    kw = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, dims=dims, base=rng.choice([10.0, 1e4, 1e6]), scale=rng.choice([0.1, 0.35, dim ** -0.5]),
              window=rng.choice([1, 2, 5, 16, 17, 40, None]), scaling=rng.choice([None, None, banded(factor=rng.choice([2.0, 8.0]), original=rng.choice([8, 64]))]))
    if kind == "attention":
        return conv_layer(mlp=None, conv=rng.choice([1, 2, 3, 4, 6]), softcap=rng.choice([None, 4.0]), **kw)
    if kind == "attention_2":
        return keys_as_values_layer(mlp=None, softcap=rng.choice([None, 4.0, 30.0]), **kw)
    owners = [j for j, L in enumerate(earlier) if L["type"] == "attention_3" and "kv_from" not in L["mixer"]]
    if owners and rng.random() < 0.5:
        j = rng.choice(owners)
        o = earlier[j]["mixer"]
        kw.update(kv_heads=o["kv_heads"], heads=o["kv_heads"] * rng.choice([1, 2]), dim=o["dim"], vdim=o["vdim"], dims=o["rot"]["dims"],
                  base=o["rot"]["base"], scaling=o["rot"].get("scaling"))
        return sink_layer(mlp=None, softcap=rng.choice([None, 6.0]), kv_from=j, **kw)
    return sink_layer(mlp=None, softcap=rng.choice([None, 6.0]), **kw)


def random_model(rng):
    layers = []
    for i in range(rng.randint(1, 5)):
        layer = random_mixer(rng, i, layers)
        layer["mlp"] = rng.choice([None, dense(ff=rng.choice([8, 24, 50])),
                                   experts(ff=rng.choice([8, 12, 32]), experts=rng.choice([1, 2, 5, 9]), top=1, shared=rng.choice([0, 8, 20]))])
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = rng.randint(1, layer["mlp"]["router"]["experts"])
        layers.append(layer)
    return model_config(layers, width=rng.choice([16, 24, 40, 64, 66]), vocab=rng.choice([37, 100, 257]), eps=rng.choice([1e-6, 1e-5, 1e-3]),
                        scale=rng.choice([1.0, 3.0, 9.5]), softcap=rng.choice([None, 5.0, 30.0]))


@pytest.mark.parametrize("seed", range(16))
def test_random_models_and_schedules(tmp_path, seed):
    rng = random.Random(900 + seed)
    cfg = random_model(rng)
    folder = make_folder(tmp_path, cfg, seed=seed)
    requests = {f"r{i}": tokens(seed * 10 + i, rng.randint(1, 90), cfg["vocab"]) for i in range(rng.randint(2, 5))}
    ref = reference(folder, requests)
    page_size = rng.choice([1, 2, 8, 16, 32])
    regime = rng.choice(["mixed", "portions", "tail"])
    steps = {"mixed": lambda: rc.mixed(requests, live=rng.randint(2, 4), portion=rng.randint(2, 20), decode_after=rng.choice([0.4, 0.8])),
             "portions": lambda: rc.changing_portions(requests, sizes=tuple(rng.randint(2, 17) for _ in range(7))),
             "tail": lambda: rc.tail_one_by_one(requests, tail=rng.randint(1, 30))}[regime]()
    for dtype in ("float32", "bfloat16"):
        got = run_steps(folder, dtype, steps, page_size, pool_tokens=rc.tokens_needed(steps, round_to=max(page_size, 4)))
        alone = run_steps(folder, dtype, rc.whole(requests), page_size)
        for rid in requests:
            assert agrees(got[rid], ref[rid], dtype), (cfg, page_size, regime, dtype, rid, distance(got[rid], ref[rid]))
            if dtype == "float32":
                assert torch.equal(got[rid], alone[rid]), (cfg, page_size, regime, rid)


def test_a_model_of_middling_sizes(tmp_path):
    """Sizes beyond the tiny ones: heads of 64 and 128 (the cache's swizzled tiles), values of another size than keys, eight
    query heads per key head, windows of several pages, nine experts of which three are named, a prompt long enough for
    the grouped product, and portions beside decoded tokens of other requests."""
    cfg = model_config([keys_as_values_layer(heads=8, kv_heads=2, dim=64, vdim=64, dims=32, window=100, scale=0.1, softcap=20.0, mlp=dense(ff=256)),
                        sink_layer(heads=8, kv_heads=1, dim=128, vdim=64, dims=64, base=1e4, window=70, scale=0.08, scaling=banded(8.0, 1.0, 4.0, 128),
                                   mlp=experts(ff=96, experts=9, top=3, shared=64)),
                        conv_layer(heads=6, kv_heads=3, dim=32, vdim=48, dims=16, base=1e6, window=150, scale=0.17, conv=4,
                                   mlp=experts(ff=64, experts=4, top=2, shared=0)),
                        sink_layer(heads=16, kv_heads=1, dim=128, vdim=64, dims=64, base=1e4, window=200, scale=0.08, scaling=banded(8.0, 1.0, 4.0, 128),
                                   kv_from=1, mlp=None)],
                       width=384, vocab=700, softcap=30.0, scale=8.0)
    folder = make_folder(tmp_path, cfg, std=0.04)
    requests = {"a": tokens(71, 420, 700), "b": tokens(72, 130, 700), "c": tokens(73, 67, 700)}
    ref = reference(folder, requests)
    for dtype in ("float32", "bfloat16"):
        for steps in (rc.whole(requests), rc.mixed(requests, live=3, portion=40, decode_after=0.8)):
            got = run_steps(folder, dtype, steps, page_size=16)
            for rid in requests:
                assert agrees(got[rid], ref[rid], dtype), (dtype, rid, distance(got[rid], ref[rid]))


# ----------------------------------------------------------------------------- through the engine's entry point
@pytest.mark.parametrize("options", [dict(), dict(cuda_graph=False, overlap_schedule=False), dict(max_num_batched_tokens=16, max_num_seqs=2)])
def test_greedy_generation_through_the_engine(tmp_path, options):
    from tandem_b200.engine.llm_engine import LLM
    from tandem_b200.sampling.params import SamplingParams

    folder = make_folder(tmp_path, HYBRID)
    prompts = [tokens(51, 23), tokens(52, 5), tokens(53, 40)]
    cfg, w = plain.read_folder(folder)
    llm = LLM(folder, dtype="float32", block_size=4, num_kv_blocks=64, **options)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        seq = list(prompt)
        for produced in out.output_token_ids:
            logits = plain.forward(cfg, w, seq)[0][-1]
            best = int(logits.argmax())
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) > 1e-3:  # a tie within rounding may go either way
                assert produced == best, (len(seq) - len(prompt))
            seq.append(produced)
        assert len(out.output_token_ids) == 12
    assert llm.engine.cache.all_free()


def test_decoding_under_cuda_graphs_in_bfloat16(tmp_path):
    """The same greedy tokens with captured decode steps as without."""
    from tandem_b200.engine.llm_engine import LLM
    from tandem_b200.sampling.params import SamplingParams

    folder = make_folder(tmp_path, HYBRID)
    prompts = [tokens(54, 19), tokens(55, 3), tokens(56, 33), tokens(57, 8)]
    outs = []
    for graphs in (True, False):
        llm = LLM(folder, dtype="bfloat16", block_size=16, num_kv_blocks=32, cuda_graph=graphs)
        outs.append([o.output_token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True))])
        del llm
    assert outs[0] == outs[1]


def test_the_trace_program_replays_a_recorded_run(tmp_path):
    """``bin/trace_run`` on a trace of mixed steps: the logits it writes are the plain ones."""
    import subprocess
    import sys

    folder = make_folder(tmp_path, HYBRID)
    requests = {"a": tokens(61, 70), "b": tokens(62, 9), "c": tokens(63, 31)}
    ref = reference(folder, requests)
    steps = rc.mixed(requests, live=3, portion=7, decode_after=0.6)
    out_dir = os.path.join(str(tmp_path), "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
                          "--max-tokens", str(rc.tokens_needed(steps, round_to=64))],
                         input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(-1, VOCAB).astype(np.float64)
               for s in steps if any(e["want"] for e in s["entries"])}
    got = {rid: torch.from_numpy(np.stack(rows)) for rid, rows in rc.collect(steps, outputs).items()}
    for rid in requests:
        assert distance(got[rid], ref[rid]) < LIMIT["float32"], rid


def test_the_command_line_makes_a_model_and_generates(tmp_path):
    """``tandem random-model`` writes a folder from the configuration file alone, ``tandem generate`` picks the model class by
    that file, samples greedily and with a seeded temperature, and records its steps; the greedy tokens are the plain ones."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tandem = [sys.executable, os.path.join(root, "bin", "tandem")]
    cfg_path = os.path.join(str(tmp_path), "cfg.json")
    with open(cfg_path, "w", encoding="utf-8") as f:
        json.dump(HYBRID, f)
    folder = os.path.join(str(tmp_path), "made")
    made = subprocess.run(tandem + ["random-model", "--config", cfg_path, "--out", folder, "--seed", "4"], capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    cfg, w = plain.read_folder(folder)
    assert cfg["architecture"] == "Deletar" and w["l1.mlp.table"].dtype == torch.int32
    prompt = tokens(81, 17)
    trace = os.path.join(str(tmp_path), "run.jsonl")
    common = ["generate", "--model", folder, "--dtype", "float32", "--prompt-ids", " ".join(map(str, prompt)), "--max-tokens", "8",
              "--ignore-eos", "--block-size", "4", "--num-kv-blocks", "32"]
    run = subprocess.run(tandem + common + ["--temperature", "0", "--trace-out", trace], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    produced = [int(t) for t in run.stdout.split()]
    seq = list(prompt)
    for token in produced:
        logits = plain.forward(cfg, w, seq)[0][-1]
        top2 = logits.topk(2).values
        if float(top2[0] - top2[1]) > 1e-3:
            assert token == int(logits.argmax()), len(seq) - len(prompt)
        seq.append(token)
    assert len(produced) == 8 and os.path.getsize(trace) > 0
    sampled = [subprocess.run(tandem + common + ["--temperature", "0.9", "--top-k", "20", "--seed", "5"], capture_output=True, text=True, timeout=600)
               for _ in range(2)]
    assert sampled[0].returncode == 0 and sampled[0].stdout == sampled[1].stdout and len(sampled[0].stdout.split()) == 8
