"""Muzopel in the engine against the plain implementation (``plain_muzopel``): each mechanism alone, the kernels
alone, whole prompts against decoding and against portions, mixed batches on small pools with pages and state
rows handed on, far keys, the convolution's reach, the depth average and the identity experts made visible by
the weights, long decoding, other sizes, greedy generation through ``LLMEngine``.  Every test builds its own
tiny model with random weights."""

import json
import math
import os
import random

import numpy as np
import pytest
import torch

import plain_muzopel as plain
import replay_cases as rc

pytestmark = pytest.mark.gpu

VOCAB = 173


# ----------------------------------------------------------------------------- tiny models
def experts(ff=24, experts=5, identity=2, top=3):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top))


def stretched(factor=3.0, original=40, fast=8.0, slow=1.0):
    return dict(factor=factor, original=original, fast=fast, slow=slow)


def query_latent_layer(heads=3, dim=12, rot_dim=8, vdim=10, kv_rank=20, q_rank=28, scale=0.2, base=500.0, scaling=stretched(), mlp=experts()):
    rot = dict(dims=rot_dim, base=base)
    if scaling is not None:
        rot["scaling"] = scaling
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                                                    rot=rot), mlp=mlp)


def plain_query_layer(heads=4, dim=8, rot_dim=6, vdim=12, kv_rank=16, scale=0.25, base=1e4, mlp=experts()):
    return dict(type="latent_attention_2", mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                                                      rot=dict(dims=rot_dim, base=base)), mlp=mlp)


def model_config(layers, width=48, vocab=VOCAB, eps=1e-5, groups=3, taps=3, softcap=12.0):
    cfg = dict(architecture="Muzopel", vocab=vocab, width=width, norm=dict(eps=eps, groups=groups), canon=dict(taps=taps), layers=layers)
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


# a query-latent layer whose latent the tensor-core attention kernel takes (key 32 + 16, value 32), plain-query layers
# between, a layer without a feed-forward, five taps
HYBRID = model_config([query_latent_layer(heads=4, dim=16, rot_dim=16, vdim=8, kv_rank=32, q_rank=24), plain_query_layer(mlp=None),
                       plain_query_layer(heads=2, dim=10, rot_dim=4, vdim=6, kv_rank=12, mlp=experts(ff=16, experts=3, identity=1, top=2)),
                       query_latent_layer(mlp=experts(ff=40, experts=7, identity=0, top=1))], taps=5, groups=4)


def make_folder(tmp_path, cfg, seed=3, edits=None, name="m", std=0.08) -> str:
    """A model folder with bfloat16-representable random weights; ``edits``: tensor name -> function
    that changes the float32 tensor in place."""
    from safetensors.torch import save_file

    from tandem_b200.config.muzopel_config import MuzopelConfig
    from tandem_b200.models.muzopel import random_weights

    typed = MuzopelConfig.from_dict(json.loads(json.dumps(cfg)))
    tensors = {}
    for tensor_name, t in random_weights(typed, seed, "cpu", torch.float32, std=std):
        if edits and tensor_name in edits:
            edits[tensor_name](t)
        tensors[tensor_name] = t.to(torch.bfloat16).contiguous()
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


def close_but_for_router_flips(got, ref, share=4) -> bool:
    """bfloat16 with routed experts: the router reads rounded inputs, so among hundreds of random positions a
    few pick another expert where two scores nearly tie (with one expert chosen of two, one position in thirty).  The
    norm on the feed-forward's output makes such a choice a change of full size at that position, and the positions
    behind it see it through the cache and the convolutions, fading.  A fault of the engine shows in float32 (where
    every test demands the plain numbers) and does not fade.  At most one position in ``share`` (or one) may exceed
    the limit."""
    e = per_position(got, ref)
    return int((e > LIMIT["bfloat16"]).sum()) <= max(1, e.numel() // share)


def agrees(got, ref, dtype) -> bool:
    return close_but_for_router_flips(got, ref) if dtype == "bfloat16" else distance(got, ref) < LIMIT[dtype]


def reference(folder, requests):
    cfg, w = plain.read_folder(folder)
    return {rid: plain.forward(cfg, w, t) for rid, t in requests.items()}


# ----------------------------------------------------------------------------- each mechanism alone
ALONE = {
    "query_latent": model_config([query_latent_layer(mlp=None)]),
    "query_latent_unstretched": model_config([query_latent_layer(scaling=None, mlp=None)]),
    "query_latent_tensor_cores": model_config([query_latent_layer(heads=2, dim=24, rot_dim=16, vdim=16, kv_rank=48, q_rank=16, mlp=None)]),
    "query_latent_one_head": model_config([query_latent_layer(heads=1, dim=16, rot_dim=2, vdim=32, kv_rank=7, q_rank=5, mlp=None)]),
    "stretched_all_pairs": model_config([query_latent_layer(rot_dim=12, scaling=stretched(factor=8.0, original=16, fast=1.5, slow=1.2), mlp=None)]),
    "plain_query": model_config([plain_query_layer(mlp=None)]),
    "plain_query_many_heads": model_config([plain_query_layer(heads=12, dim=8, rot_dim=4, vdim=6, kv_rank=12, mlp=None)]),
    "one_tap": model_config([plain_query_layer(mlp=experts())], taps=1),
    "two_taps": model_config([plain_query_layer(mlp=experts())], taps=2),
    "eleven_taps": model_config([query_latent_layer(mlp=experts())], taps=11),
    "one_norm_group": model_config([plain_query_layer(mlp=None)], groups=1),
    "a_norm_group_per_number": model_config([plain_query_layer(mlp=None)], groups=48, eps=1e-2),
    "experts": model_config([plain_query_layer(mlp=experts(ff=24, experts=7, identity=0, top=3))]),
    "identity_experts": model_config([plain_query_layer(mlp=experts(ff=10, experts=2, identity=3, top=2))]),
    "one_expert_of_two": model_config([query_latent_layer(mlp=experts(ff=9, experts=1, identity=1, top=1))]),
    "all_experts_chosen": model_config([query_latent_layer(mlp=experts(ff=16, experts=3, identity=1, top=4))]),
    "no_softcap": model_config([plain_query_layer()], softcap=None),
    "depth_average": model_config([plain_query_layer(mlp=None), query_latent_layer(mlp=None), plain_query_layer()]),
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(tmp_path, name, dtype):
    folder = make_folder(tmp_path, ALONE[name])
    requests = {"a": tokens(1, 45), "b": tokens(2, 1)}
    ref = reference(folder, requests)
    got = run_steps(folder, dtype, rc.whole(requests))
    for rid in requests:
        assert agrees(got[rid], ref[rid], dtype), (name, rid, distance(got[rid], ref[rid]))


def test_the_stream_after_every_layer_is_the_plain_one(tmp_path):
    """What a layer hands on (its depth average), in float32."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry

    folder = make_folder(tmp_path, HYBRID)
    toks = tokens(5, 30)
    cfg, w = plain.read_folder(folder)
    _, layers = plain.forward(cfg, w, toks, keep_layers=True)
    decoder, _ = load_model(folder, "float32", "cuda:0")
    ex = build_executor(decoder, page_size=8, num_pages=8, max_requests=2)
    seen = []
    for layer in decoder.layers:
        inner = layer.block.forward

        def spy(l, x, residual, ctx, inner=inner):
            out = inner(l, x, residual, ctx)
            assert out is None  # everything is in the stream
            seen.append(residual.double().cpu())
            return out

        layer.block.forward = spy
    ex.step([StepEntry("a", toks, [0])], end=["a"])
    assert len(seen) == len(layers) == 4
    for i, (g, r) in enumerate(zip(seen, layers)):
        assert (g - r).abs().max() < 1e-5 * max(1.0, float(r.abs().max())), i


# ----------------------------------------------------------------------------- the kernels alone
class Batch:
    """The device arrays of a step that the kernels of the post-norm link read."""

    def __init__(self, starts, lens, slots):
        seq, pos, cu = [], [], [0]
        for b, (s, n) in enumerate(zip(starts, lens)):
            seq += [b] * n
            pos += list(range(s, s + n))
            cu.append(cu[-1] + n)
        as_int = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
        self.seq_of_token, self.positions, self.cu_seqlens = as_int(seq), as_int(pos), as_int(cu)
        self.seq_starts, self.state_slots, self.num_seqs = as_int(starts), as_int(slots), len(lens)


@pytest.mark.parametrize("W,groups,taps", [(48, 3, 3), (40, 1, 1), (64, 64, 4), (96, 4, 8), (24, 2, 2)])
def test_the_link_kernel_against_its_pieces_and_the_plain_ones(W, groups, taps):
    """x' = x + norm(y), kept, averaged over earlier results, then the next sublayer's convolution: one launch against the
    single kernels and against float64, over two requests cut into steps whose borders fall inside the convolution's reach."""
    from tandem_b200.kernels import post_norm

    g = torch.Generator().manual_seed(W + taps)
    lens_total = [23, 9]
    xs = [torch.randn(n, W, generator=g) for n in lens_total]
    ys = [torch.randn(n, W, generator=g) * 3 for n in lens_total]
    earlier = [[torch.randn(n, W, generator=g) for n in lens_total] for _ in range(2)]
    weight, coeff = torch.rand(W, generator=g) + 0.5, torch.randn(3, generator=g)
    tap_w = torch.randn(W, taps, generator=g) * 0.5
    eps = 1e-3
    want_x, want_h = [], []
    for i in range(2):
        made = xs[i].double() + plain.group_norm(ys[i].double(), weight.double(), groups, eps)
        mixed = coeff[0].double() * earlier[0][i].double() + coeff[1].double() * earlier[1][i].double() + coeff[2].double() * made
        want_x.append((made, mixed))
        want_h.append(plain.short_convolution(mixed, tap_w.double()))
    state = torch.zeros(5, max(taps - 1, 1), W).cuda() + 7.0  # rows 3 and 1 are the requests'; what is there is stale
    state[3].zero_()
    state[1].zero_()
    state_fused = state.clone()
    at = [0, 0]
    got_h, got_x, got_kept, got_h2 = [[], []], [[], []], [[], []], [[], []]
    for cut in ((1, 2), (2, 1), (5, 2), (1, 1), (14, 3)):
        b = Batch(at, list(cut), [3, 1])
        cat = lambda seqs: torch.cat([seqs[i][at[i]: at[i] + cut[i]] for i in range(2)]).cuda().contiguous()
        x, y = cat(xs), cat(ys)
        planes = torch.stack([cat(earlier[0]), cat(earlier[1]), torch.zeros_like(x)]).contiguous()
        out = torch.empty_like(x)
        h = post_norm.link(x, y, weight.cuda(), groups, eps, out, planes=planes, coeff=coeff.cuda(), n_planes=2, taps=tap_w.cuda(),
                           state=state_fused if taps > 1 else None, ctx=b, out_dtype=torch.float32)
        post_norm.short_conv_state(out, state_fused, b, taps)
        # the same from the single kernels
        stream, kept = x.clone(), torch.empty_like(x)
        post_norm.group_norm_add(y, weight.cuda(), groups, eps, stream, keep=kept)
        planes2 = torch.stack([planes[0], planes[1], kept]).contiguous()
        post_norm.depth_average(planes2, coeff.cuda(), 3, stream)
        h2 = post_norm.short_conv(stream, tap_w.cuda(), state if taps > 1 else None, b, torch.float32)
        post_norm.short_conv_state(stream, state, b, taps)
        o = 0
        for i in range(2):
            got_h[i].append(h[o: o + cut[i]].cpu())
            got_h2[i].append(h2[o: o + cut[i]].cpu())
            got_x[i].append(out[o: o + cut[i]].cpu())
            got_kept[i].append(planes[2][o: o + cut[i]].cpu())
            o += cut[i]
        at = [at[i] + cut[i] for i in range(2)]
    assert at == lens_total
    for i in range(2):
        assert (torch.cat(got_kept[i]).double() - want_x[i][0]).abs().max() < 1e-5
        assert (torch.cat(got_x[i]).double() - want_x[i][1]).abs().max() < 1e-5
        assert (torch.cat(got_h[i]).double() - want_h[i]).abs().max() < 2e-5
        assert (torch.cat(got_h2[i]).double() - want_h[i]).abs().max() < 2e-5
    assert torch.equal(state[[0, 2, 4]], torch.full_like(state[[0, 2, 4]], 7.0))  # nobody else's rows were touched
    if taps > 1:
        assert torch.equal(state, state_fused)


@pytest.mark.parametrize("W,groups,taps,y_dtype,h_dtype", [(64, 4, 4, "float32", "float32"), (1280, 5, 3, "bfloat16", "bfloat16"),
                                                          (30, 3, 6, "float32", "bfloat16"), (2304, 1, 2, "bfloat16", "float32")])
def test_the_link_over_long_runs_of_rows(W, groups, taps, y_dtype, h_dtype):
    """Steps long enough that a thread walks down several rows, with requests that begin inside a run, after a step that
    left a state: against float64, and the same bits as the same tokens one step each."""
    from tandem_b200.kernels import post_norm

    g = torch.Generator().manual_seed(W)
    yt, ht = getattr(torch, y_dtype), getattr(torch, h_dtype)
    lens = [700, 3, 1, 650, 2]
    first = [2, 0, 0, 1, 0]  # tokens that an earlier step brought
    total = [a + b for a, b in zip(lens, first)]
    xs = [torch.randn(n, W, generator=g) for n in total]
    ys = [(torch.randn(n, W, generator=g) * 2).to(yt) for n in total]
    weight, tap_w = torch.rand(W, generator=g) + 0.5, torch.randn(W, taps, generator=g) * 0.4
    eps = 1e-4
    want_x = [x.double() + plain.group_norm(y.double(), weight.double(), groups, eps) for x, y in zip(xs, ys)]
    want_h = [plain.short_convolution(x, tap_w.double()) for x in want_x]

    def run(steps):
        """steps: lists of (request, begin, count); -> per request x_out and h rows in order."""
        state = torch.full((6, taps - 1, W), 5.0).cuda()
        state[:5].zero_()
        got_x, got_h = [[] for _ in lens], [[] for _ in lens]
        for step in steps:
            b = Batch([s for _, s, _ in step], [n for _, _, n in step], [i for i, _, _ in step])
            x = torch.cat([xs[i][s: s + n] for i, s, n in step]).cuda()
            y = torch.cat([ys[i][s: s + n] for i, s, n in step]).cuda()
            out = torch.empty_like(x)
            h = post_norm.link(x, y, weight.cuda(), groups, eps, out, taps=tap_w.cuda(), state=state, ctx=b, out_dtype=ht)
            post_norm.short_conv_state(out, state, b, taps)
            o = 0
            for i, _, n in step:
                got_x[i].append(out[o: o + n].cpu())
                got_h[i].append(h[o: o + n].cpu())
                o += n
        assert float(state[5].min()) == 5.0
        return [torch.cat(v) if v else None for v in got_x], [torch.cat(v) if v else None for v in got_h]

    early = [(i, 0, n) for i, n in enumerate(first) if n]
    big_x, big_h = run([early, [(i, first[i], lens[i]) for i in range(5)]])
    for i in range(5):
        assert (big_x[i].double() - want_x[i]).abs().max() < 2e-5
        scale = 2.0 ** -7 if h_dtype == "bfloat16" else 1e-5
        assert (big_h[i].double() - want_h[i]).abs().max() < scale * max(1.0, float(want_h[i].abs().max()))
    short = [0, 3]  # one token a step for the head of a long request and a whole short one, which is enough for every tap
    one_x, one_h = run([early] + [[(i, t, 1)] for i in short for t in range(first[i], min(total[i], first[i] + 12))])
    for i in short:
        n = min(total[i], first[i] + 12)
        assert torch.equal(one_x[i], big_x[i][:n]) and torch.equal(one_h[i], big_h[i][:n])


def test_a_rows_scale_does_not_depend_on_where_the_row_lies():
    """Rows cut out of a wider array start on any address; their norm is the same bits as that of a copy."""
    from tandem_b200.kernels import post_norm

    g = torch.Generator().manual_seed(4)
    for W, groups, off in ((64, 4, 3), (30, 3, 1), (130, 1, 2)):
        wide = (torch.randn(9, W + 7, generator=g) * 3).cuda()
        w = (torch.rand(W, generator=g) + 0.5).cuda()
        view = wide[:, off: off + W]
        a = post_norm.group_norm(view, w, groups, 1e-5, torch.float32)
        b = post_norm.group_norm(view.contiguous(), w, groups, 1e-5, torch.float32)
        assert torch.equal(a, b)
        want = plain.group_norm(view.double().cpu(), w.double().cpu(), groups, 1e-5)
        assert (a.cpu().double() - want).abs().max() < 1e-5
        inv = post_norm.row_scales(view.contiguous(), groups, 1e-5).cpu().double()
        rms = view.double().cpu().view(9, groups, W // groups).pow(2).mean(-1).add(1e-5).rsqrt()
        assert (inv - rms).abs().max() < 1e-5 * float(rms.max())


def test_the_grouped_norm_gathers_rows_and_rounds_once():
    from tandem_b200.kernels import post_norm

    g = torch.Generator().manual_seed(9)
    x = torch.randn(11, 60, generator=g) * 4
    w = torch.rand(60, generator=g) + 0.5
    rows = torch.tensor([10, 0, 3], dtype=torch.int32)
    for groups in (1, 4, 5, 60):
        want = plain.group_norm(x.double(), w.double(), groups, 1e-4)
        got = post_norm.group_norm(x.cuda(), w.cuda(), groups, 1e-4, torch.float32, rows=rows.cuda()).cpu().double()
        assert (got - want[rows.long()]).abs().max() < 1e-5
        half = post_norm.group_norm(x.cuda(), w.cuda(), groups, 1e-4, torch.bfloat16).cpu()
        assert torch.equal(half, post_norm.group_norm(x.cuda(), w.cuda(), groups, 1e-4, torch.float32).cpu().to(torch.bfloat16))
        wide = torch.cat([x, x], 1).cuda()  # rows of a wider tensor: the norm's input is a view
        part = post_norm.group_norm(wide[:, 60:], w.cuda(), groups, 1e-4, torch.float32).cpu().double()
        assert (part - want).abs().max() < 1e-5


@pytest.mark.parametrize("top,real,identity,ff,width", [(2, 6, 0, 24, 64), (1, 2, 1, 40, 48), (4, 6, 3, 16, 96), (3, 1, 2, 8, 64)])
def test_the_expert_kernels_without_a_gate_and_with_identity_experts(top, real, identity, ff, width):
    """Routing with a bias on the choice against the plain choice; the kernel of one warp per output, the sorted tiles on
    mma.sync and the grouped tcgen05 product against float64, for token counts around a tile's edge."""
    from tandem_b200.kernels import moe

    g = torch.Generator().manual_seed(top + real)
    E = real + identity
    for T in (1, 5, 63, 64, 65, 200, 300, 700):
        x = torch.randn(T, width, generator=g).to(torch.bfloat16)
        up = (torch.randn(real, ff, width, generator=g) * 0.2).to(torch.bfloat16)
        down = (torch.randn(real, width, ff, generator=g) * 0.2).to(torch.bfloat16)
        logits = torch.randn(T, E, generator=g) * 2
        bias = torch.randn(E, generator=g) * 0.3
        ids, weights = moe.route(logits.cuda(), top, "softmax", False, 1.0, bias.cuda())
        s = torch.softmax(logits.double(), -1)
        _, idx = torch.topk(s + bias.double(), top, dim=-1)
        assert torch.equal(ids.cpu().long().sort(-1).values, idx.sort(-1).values)
        assert (weights.cpu().double().sort(-1).values - torch.gather(s, 1, idx).sort(-1).values).abs().max() < 1e-6
        ref = torch.zeros(T, width, dtype=torch.float64)
        ids_host, weights_host = ids.cpu(), weights.cpu().double()
        for e in range(E):
            rows, ks = (ids_host == e).nonzero(as_tuple=True)
            if len(rows):
                xe = x[rows].double()
                out = xe if e >= real else plain.gelu_erf(xe @ up[e].double().T) @ down[e].double().T
                ref.index_add_(0, rows, weights_host[rows, ks][:, None] * out)
        scale = float(ref.abs().max())
        for mode in ("simt", "tiles", "wide"):
            os.environ["TANDEM_MOE"] = mode
            try:
                got = moe.experts(x.cuda(), up.cuda(), down.cuda(), ids, weights, gated=False, num_router_outputs=E).cpu().double()
            finally:
                os.environ.pop("TANDEM_MOE", None)
            assert (got - ref).abs().max() < 2e-2 * scale, (mode, T)
        got = moe.experts(x.float().cuda(), up.float().cuda(), down.float().cuda(), ids, weights, gated=False, num_router_outputs=E).cpu().double()
        assert (got - ref).abs().max() < 1e-5 * scale, T


def test_the_choice_bias_changes_the_choice_and_not_the_weight():
    from tandem_b200.kernels import moe

    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).cuda()
    bias = torch.tensor([0.0, 0.0, 0.0, 5.0]).cuda()
    ids, weights = moe.route(logits, 2, "softmax", False, 1.0, bias)
    s = torch.softmax(logits.double().cpu(), -1)[0]
    assert ids.cpu().tolist() == [[3, 0]]
    assert abs(float(weights[0, 0]) - float(s[3])) < 1e-7 and abs(float(weights[0, 1]) - float(s[0])) < 1e-7
    ids, _ = moe.route(logits, 2, "softmax", False, 1.0, None)
    assert ids.cpu().tolist() == [[0, 1]]


def test_the_rotation_of_interleaved_pairs_with_stretched_frequencies():
    """The cache entry and the queries' rotated part as the kernel writes them, against the plain rotation: pairs (2 i, 2 i + 1),
    stretched frequencies, cos and sin times the factor, numbers beyond the rotated ones untouched, positions in the thousands."""
    from tandem_b200.config.plan import RotaryScalingSpec, rotary_table
    from tandem_b200.kernels import latent_attention as kernels
    from tandem_b200.parts.base import KVView

    g = torch.Generator().manual_seed(2)
    T, H, d, r, rd, R, page = 7, 3, 5, 10, 6, 9, 4
    rot = dict(dims=rd, base=300.0, scaling=stretched(factor=5.0, original=64, fast=6.0, slow=0.7))
    freq, mag = rotary_table(rd, 300.0, RotaryScalingSpec(5.0, 64, 6.0, 0.7))
    want_f, want_mag = plain.rotary_frequencies(rot)
    assert abs(mag - want_mag) < 1e-12 and (torch.tensor(freq, dtype=torch.float64) - want_f).abs().max() < 1e-15
    assert not torch.equal(want_f, plain.rotary_frequencies(dict(dims=rd, base=300.0))[0])
    positions = torch.tensor([0, 1, 2, 3001, 3002, 17, 4], dtype=torch.int32)
    q = torch.randn(T, H * (d + r), generator=g)
    proj = torch.randn(T, 3 + R + r, generator=g)  # the down-projection from column 3
    norm_w = torch.rand(R, generator=g) + 0.5
    k_cache, v_cache = torch.zeros(2, 1, page, R + r).cuda(), torch.zeros(2, 1, page, R).cuda()
    slots = torch.tensor([0, 1, 2, 3, 4, 5, 7], dtype=torch.int32).cuda()
    kv = KVView(k_cache, v_cache, None, slots, page, True)
    out = kernels.prepare(proj.cuda(), 3, norm_w.cuda(), torch.tensor(freq, dtype=torch.float32).cuda(), positions.cuda(), kv, H, d, r, R, 1e-5,
                          queries=q.cuda(), interleaved=True, magnitude=mag).cpu().double()
    q_rot = plain.rotate_pairs(q.double().view(T, H, d + r)[..., d:].transpose(0, 1), positions, rot).transpose(0, 1)
    assert (out[..., R:] - q_rot).abs().max() < 2e-4  # angles are float32: position 3002 times a frequency near one
    assert torch.equal(out[..., R + rd:], q.double().view(T, H, d + r)[..., d + rd:])
    latent = plain.unit_rms(proj[:, 3: 3 + R].double(), 1e-5) * norm_w.double()
    k_rot = plain.rotate_pairs(proj[:, 3 + R:].double(), positions, rot)
    rows = k_cache.view(-1, R + r)[slots.long()].cpu().double()
    assert (rows[:, :R] - latent).abs().max() < 1e-5 and (rows[:, R:] - k_rot).abs().max() < 2e-4
    assert (v_cache.view(-1, R)[slots.long()].cpu().double() - latent).abs().max() < 1e-5
    assert float(k_cache.view(-1, R + r)[6].abs().max()) == 0.0


def test_a_gate_per_head():
    from tandem_b200.kernels import latent_attention as kernels

    g = torch.Generator().manual_seed(3)
    o, gate = torch.randn(5, 12, generator=g), torch.randn(5, 7, generator=g)
    got = kernels.sigmoid_gate(o.cuda(), gate.cuda()[:, 2:5], torch.float32, per=4).cpu()
    want = o.view(5, 3, 4) * torch.sigmoid(gate[:, 2:5])[:, :, None]
    assert (got.view(5, 3, 4) - want).abs().max() < 1e-6


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
    """Portions shorter than the convolution's reach (five taps): its inputs come from the state and from the step."""
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
    alone = run_steps(folder, dtype, rc.whole(requests), 4) if dtype == "float32" else None
    for rid in requests:
        assert agrees(got[rid], ref[rid], dtype), rid
        if alone is not None:
            assert torch.equal(got[rid], alone[rid]), rid


def test_a_state_row_that_is_used_again_starts_from_zero(tmp_path):
    """One row for all: the second request finds the first one's convolution inputs there, in every layer and for both sublayers."""
    folder = make_folder(tmp_path, model_config([plain_query_layer(), query_latent_layer()], taps=4))
    requests = {"first": tokens(1, 40), "second": tokens(2, 25), "third": tokens(3, 2), "fourth": tokens(4, 1)}
    ref = reference(folder, requests)
    got = run_steps(folder, "float32", rc.tail_one_by_one(requests, tail=5), page_size=8, max_requests=1)
    for rid in requests:
        assert distance(got[rid], ref[rid]) < LIMIT["float32"], rid


def test_long_decoding(tmp_path):
    """Three hundred tokens one by one: page after page of latents, the convolutions' inputs carried all the way."""
    folder = make_folder(tmp_path, model_config([query_latent_layer(), plain_query_layer(mlp=None),
                                                 query_latent_layer(heads=4, dim=16, rot_dim=16, vdim=8, kv_rank=32, q_rank=40)]))
    requests = {"a": tokens(21, 330)}
    ref = reference(folder, requests)
    for dtype in ("float32", "bfloat16"):
        got = run_steps(folder, dtype, rc.tail_one_by_one(requests, tail=300), page_size=8)
        assert agrees(got["a"], ref["a"], dtype), dtype


# ----------------------------------------------------------------------------- faults made visible
def zero(t):
    t.zero_()


def quiet(t):
    t.mul_(0.02)


@pytest.mark.parametrize("kind", ["latent_attention", "latent_attention_2"])
def test_one_far_key_among_hundreds(tmp_path, kind):
    """The rotated key part of one early token and the rotated query part of the last tokens are made loud along a
    pair that turns slowly, so that the last tokens look far back across many pages; prompt, portions and single
    tokens.  The convolution in front of the mixer is switched off so that a token's key is its own.  The oracle
    itself tells a sequence apart in which that key is not there."""
    H, d, r, R, vocab = 2, 8, 4, 16, 60
    if kind == "latent_attention":
        layer = query_latent_layer(heads=H, dim=d, rot_dim=r, vdim=8, kv_rank=R, q_rank=48, scale=1.0, base=1e9, scaling=None, mlp=None)
    else:
        layer = plain_query_layer(heads=H, dim=d, rot_dim=r, vdim=8, kv_rank=R, scale=1.0, base=1e9, mlp=None)
    cfg = model_config([layer], vocab=vocab, width=48)
    folder = make_folder(tmp_path, cfg, edits={"l0.canon1": zero})
    _, w = plain.read_folder(folder)
    toks = tokens(5, 520, vocab)
    far, key_token, query_token = 13, 59, 58
    toks = [0 if t in (key_token, query_token) else t for t in toks]
    toks[far] = key_token
    for i in range(470, 520):
        toks[i] = query_token
    h_key = plain.group_norm(w["embed"][key_token], w["embed.norm"], 3, 1e-5)
    h_query = plain.group_norm(w["embed"][query_token], w["embed.norm"], 3, 1e-5)

    def loud_key(t):  # number 2 of the rotated part: pair 1, which turns by base^(-1/2) a position, hardly at all
        quiet(t)
        t[R + 2] += (6.0 * h_key / (h_key @ h_key)).float()

    edits = {"l0.canon1": zero, "l0.mix.dkv": loud_key}
    if kind == "latent_attention":  # the query's latent is normed: a loud direction in it, and its expansion to every head's rotated number 2
        def loud_latent(t):
            quiet(t)
            t[0] += (6.0 * h_query / (h_query @ h_query)).float()

        def expand(t):
            quiet(t)
            for head in range(H):
                t[head * (d + r) + d + 2, 0] += 1.0

        edits.update({"l0.mix.dq": loud_latent, "l0.mix.uq": expand})
    else:
        def loud_query(t):
            quiet(t)
            for head in range(H):
                t[head * (d + r) + d + 2] += (6.0 * h_query / (h_query @ h_query)).float()

        edits["l0.mix.q"] = loud_query
    folder = make_folder(tmp_path, cfg, edits=edits, name="loud")
    requests = {"a": toks}
    ref = reference(folder, requests)
    hidden = list(toks)
    hidden[far] = 0
    assert distance(reference(folder, {"a": hidden})["a"][480:], ref["a"][480:]) > 0.05  # the far key matters
    for dtype in ("float32", "bfloat16"):
        for steps in (rc.whole(requests), rc.tail_one_by_one(requests, 45), rc.changing_portions(requests, (37, 2, 64, 3))):
            got = run_steps(folder, dtype, steps, page_size=16)
            assert distance(got["a"], ref["a"]) < LIMIT[dtype], dtype


def test_the_convolutions_oldest_tap_and_no_further(tmp_path):
    """All weight on the oldest tap, in front of the mixer and in front of the feed-forward: a sublayer's input is its own
    token plus what came taps - 1 places earlier, in prompts, across portion borders and token by token; a model with
    one tap more or less is another model."""
    taps = 4

    def oldest_only(t):
        t.zero_()
        t[:, 0] = 1.5

    cfg = model_config([plain_query_layer(mlp=experts(ff=16, experts=3, identity=1, top=2))], taps=taps)
    folder = make_folder(tmp_path, cfg, edits={"l0.canon1": oldest_only, "l0.canon2": oldest_only})
    requests = {"a": tokens(31, 41), "b": tokens(32, 3), "c": tokens(33, 4)}
    ref = reference(folder, requests)
    for dtype in ("float32", "bfloat16"):
        for steps in (rc.whole(requests), rc.tail_one_by_one(requests, 30), rc.changing_portions(requests, (2,)),
                      rc.changing_portions(requests, (3, 5, 2)), rc.mixed(requests, live=3, portion=3, decode_after=0.5)):
            got = run_steps(folder, dtype, steps, page_size=4)
            for rid in requests:
                assert agrees(got[rid], ref[rid], dtype), (dtype, rid)
    cfg_read, w = plain.read_folder(folder)
    for other in (taps - 1, taps + 1):
        w2 = dict(w)
        for name in ("l0.canon1", "l0.canon2"):
            w2[name] = torch.zeros(w[name].shape[0], other, dtype=torch.float64)
            w2[name][:, 0] = 1.5
        assert distance(plain.forward(cfg_read, w2, requests["a"]), ref["a"]) > 0.05, other


def test_the_depth_average_reaches_back_to_the_embedding(tmp_path):
    """The last layer hands on mostly the embedding's rows and the first layer's result: the logits then follow them, and a
    model that averaged over the newest results only would be another model."""
    cfg = model_config([plain_query_layer(mlp=None), query_latent_layer(mlp=None), plain_query_layer(mlp=None)])

    def mostly_old(t):
        t.copy_(torch.tensor([1.5, -0.75, 0.125, 0.25]))

    folder = make_folder(tmp_path, cfg, edits={"l2.dwa": mostly_old})
    requests = {"a": tokens(41, 37), "b": tokens(42, 6)}
    ref = reference(folder, requests)
    cfg_read, w = plain.read_folder(folder)
    w2 = dict(w)
    w2["l2.dwa"] = torch.tensor([0.0, 0.0, 0.125, 0.25], dtype=torch.float64)
    assert distance(plain.forward(cfg_read, w2, requests["a"]), ref["a"]) > 0.05
    for dtype in ("float32", "bfloat16"):
        for steps in (rc.whole(requests), rc.tail_one_by_one(requests, 20), rc.mixed(requests, live=2, portion=5, decode_after=0.5)):
            got = run_steps(folder, dtype, steps, page_size=4)
            for rid in requests:
                assert distance(got[rid], ref[rid]) < LIMIT[dtype], (dtype, rid)


def test_identity_experts_that_are_always_chosen(tmp_path):
    """A large correction on the identity outputs: every token takes both of them (their weights stay the small scores), and
    one real expert; a model without the correction chooses otherwise."""
    cfg = model_config([plain_query_layer(mlp=experts(ff=16, experts=4, identity=2, top=3))])

    def prefer_identity(t):
        t.zero_()
        t[4:] = 3.0

    folder = make_folder(tmp_path, cfg, edits={"l0.mlp.correction": prefer_identity})
    requests = {"a": tokens(43, 50), "b": tokens(44, 3)}
    ref = reference(folder, requests)
    cfg_read, w = plain.read_folder(folder)
    w2 = dict(w)
    w2["l0.mlp.correction"] = torch.zeros(6, dtype=torch.float64)
    assert distance(plain.forward(cfg_read, w2, requests["a"]), ref["a"]) > 0.02
    for dtype in ("float32", "bfloat16"):
        for steps in (rc.whole(requests), rc.changing_portions(requests, (2, 9))):
            got = run_steps(folder, dtype, steps, page_size=4)
            for rid in requests:
                assert agrees(got[rid], ref[rid], dtype), (dtype, rid)


# ----------------------------------------------------------------------------- other sizes
def random_model(rng: random.Random) -> dict:
    groups = rng.choice([1, 2, 3, 4, 6])
    width = groups * rng.choice([4, 8, 10, 16, 22])
    layers = []
    for _ in range(rng.randint(1, 5)):
        mlp = None
        if rng.random() < 0.75:
            real, identity = rng.randint(1, 9), rng.choice([0, 0, 1, 2, 4])
            mlp = experts(ff=rng.choice([6, 8, 24, 40, 50]), experts=real, identity=identity, top=rng.randint(1, min(5, real + identity)))
        dim, rot = rng.choice([4, 8, 16, 24, 64]), rng.choice([2, 4, 8, 16, 32])
        sizes = dict(heads=rng.choice([1, 2, 3, 5, 8, 16]), dim=dim, rot_dim=rot, vdim=rng.choice([4, 8, 20, 64]),
                     kv_rank=rng.choice([8, 16, 24, 48, 50, 96]), scale=rng.choice([(dim + rot) ** -0.5, 0.1, 0.5]),
                     base=rng.choice([50.0, 1e4, 1e6]), mlp=mlp)
        if rng.random() < 0.5:
            scaling = rng.choice([None, stretched(factor=rng.choice([2.0, 4.0, 16.0]), original=rng.choice([16, 64, 512]),
                                                  fast=rng.choice([4.0, 32.0]), slow=rng.choice([0.5, 1.0, 2.0]))])
            layers.append(query_latent_layer(q_rank=rng.choice([6, 16, 40, 72]), scaling=scaling, **sizes))
        else:
            layers.append(plain_query_layer(**sizes))
    return model_config(layers, width=width, vocab=rng.randint(50, 400), eps=rng.choice([1e-6, 1e-5, 1e-3]), groups=groups,
                        taps=rng.choice([1, 2, 3, 4, 5, 9]), softcap=rng.choice([None, 5.0, 30.0]))


@pytest.mark.parametrize("seed", range(14))
def test_random_models_and_schedules(tmp_path, seed):
    rng = random.Random(500 + seed)
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
            else:  # the schedule against the whole prompt, both rounded alike: closer than either is to the plain numbers
                assert close_but_for_router_flips(got[rid], alone[rid], share=10), (cfg, page_size, regime, rid)


def test_a_model_of_middling_sizes(tmp_path):
    """Sizes beyond the tiny ones: a latent wider than the tensor-core tile kernel takes (keys of 160 + 32, values of 160), sixteen
    heads over the one key head, nine experts and two identity experts of which three are chosen, a prompt long enough for the
    grouped product, and portions beside decoded tokens of other requests."""
    cfg = model_config([query_latent_layer(heads=16, dim=32, rot_dim=32, vdim=24, kv_rank=160, q_rank=192, scale=0.07, base=1e5,
                                           scaling=stretched(factor=4.0, original=128, fast=16.0, slow=1.0), mlp=experts(ff=96, experts=9, identity=2, top=3)),
                        plain_query_layer(heads=8, dim=48, rot_dim=16, vdim=32, kv_rank=112, scale=0.09, base=1e4, mlp=experts(ff=64, experts=4, identity=0, top=2)),
                        plain_query_layer(heads=6, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=0.1, base=1e6, mlp=None)],
                       width=384, vocab=700, groups=4, taps=3, softcap=30.0)
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
            logits = plain.forward(cfg, w, seq)[-1]
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
