"""The Sapatar decoder in the engine against the plain implementation (tests/plain_sapatar.py): every mechanism
alone, then whole models under every way of cutting and batching the work, in float32 and bfloat16.  The tiny
models and their weights are made here."""
import numpy as np
import pytest
import torch

import plain_sapatar as plain
from helpers import (max_live_tokens, random_tokens, replay_in_process, schedule_mixed, schedule_portions, schedule_tail,
                     schedule_whole)
from test_gpu_linurax import close, ctx_of, fill
from tiny_sapatar import (SAPATAR_CONFIGS, SAPATAR_E, SAPATAR_PAGE, SAPATAR_SEEDS, SAPATAR_STD, left, moe, parallel, retention,
                          right, wkv)

import tessweave_engine_b200 as tw
from tessweave_engine_b200.csrc import ops
from tessweave_engine_b200.parts import PartSpec, Runtime, SeveralViews, StateView, build_part, dense_delta

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def named(weights, prefix="p"):
    return {f"{prefix}.{k}": v for k, v in weights.items()}


def step_ctx(rt, plan, at):
    """A StepContext for ``plan`` = [(slot, rows)] with the requests' earlier lengths in ``at`` (slot -> tokens held)."""
    positions, seq_of, slots, starts, lens, kv = [], [], [], [], [], []
    for slot, n in plan:
        if not n:
            continue
        seq_of += [len(slots)] * n
        positions += list(range(at[slot], at[slot] + n))
        starts.append(sum(lens)); lens.append(n); slots.append(slot); kv.append(at[slot] + n)
    return ctx_of(rt, positions, seq_of, slots, starts, lens, kv)


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,dims,theta", [(16, 8, 1e3), (24, 24, 5e4), (64, 2, 3e6), (32, 0, 1e4), (40, 40, 3e4)])
def test_rotation_of_halves_over_part_of_a_head(dtype, head_dim, dims, theta):
    """Value i turns with value i + dims/2; the rest of a head and the heads behind stay."""
    rt = Runtime(torch.device("cuda"), dtype)
    rope = build_part("position", PartSpec("rope", {"theta": theta, "dims": dims}), rt)
    positions = [0, 1, 2, 700, 3, 15, 16, 4095]
    ctx = ctx_of(rt, positions, [0, 0, 0, 1, 2, 2, 2, 3], [0, 1, 2, 3], [0, 3, 4, 7], [3, 1, 3, 1], [3, 701, 17, 4096])
    heads, extra = 5, 2
    x = torch.randn(len(positions), (heads + extra) * head_dim, generator=torch.Generator().manual_seed(4)).to(dtype)
    qk = x.cuda().clone()
    rope.apply(ctx, qk, heads, head_dim)
    ref = x.float().reshape(len(positions), heads + extra, head_dim)
    want = plain.rotate_half_layout(ref[:, :heads].double(), torch.tensor(positions), dims, theta).float()
    got = qk.float().cpu().reshape(len(positions), heads + extra, head_dim)
    close(got[:, :heads], want, dtype, "rotation", f32=2e-4)      # fp32 angles of positions in the thousands
    assert torch.equal(got[:, heads:], ref[:, heads:])
    assert torch.equal(got[:, :heads, dims:], ref[:, :heads, dims:])
    assert (rope.fused_rotary_table(head_dim) is not None) == (dims == head_dim)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("copies,width", [(1, 40), (2, 36), (4, 200), (8, 1000), (11, 72)])
def test_hyper_connection_pass(dtype, copies, width):
    """Start from a row, write a sub-layer's output, read the next sub-layer's input, sum the copies: each alone
    and all in one call."""
    g = torch.Generator().manual_seed(copies)
    rows = 5
    w = {"p.in": torch.randn(copies, generator=g), "p.out": torch.randn(copies, generator=g),
         "p.mix": torch.eye(copies) + 0.3 * torch.randn(copies, copies, generator=g)}
    norm_w = 1 + 0.2 * torch.randn(width, generator=g)
    x0 = torch.randn(rows, width, generator=g) * 3
    y = (torch.randn(rows, width, generator=g) * 2).to(dtype)
    dev = {k: v.cuda() for k, v in w.items()}
    streams = torch.full((rows, copies, width), float("nan"), device="cuda")
    h = torch.full((rows, width), float("nan"), dtype=dtype, device="cuda")
    ops.hyper_step(streams, rows, init=x0.cuda(), in_coef=dev["p.in"], norm_weight=norm_w.cuda(), eps=1e-5, h_out=h)
    ref = torch.stack([x0] * copies)
    assert torch.equal(streams.cpu().transpose(0, 1), ref)
    close(h.float().cpu(), plain.rms(plain.hyper_read(ref, w, "p"), norm_w, 1e-5), dtype, "first read", bf16=1e-2)
    total = torch.full((rows, width), float("nan"), device="cuda")
    ops.hyper_step(streams, rows, y=y.cuda(), mix=dev["p.mix"], out_coef=dev["p.out"], in_coef=dev["p.in"],
                   norm_weight=norm_w.cuda(), eps=1e-5, h_out=h, sum_out=total)
    ref = plain.hyper_write(ref, y.float(), w, "p")
    close(streams.cpu().transpose(0, 1), ref, torch.float32, "write", f32=3e-6)
    close(h.float().cpu(), plain.rms(plain.hyper_read(ref, w, "p"), norm_w, 1e-5), dtype, "read behind a write", bf16=1e-2)
    close(total.cpu(), ref.sum(0), torch.float32, "sum", f32=3e-6)


def run_state_mixer(rt, mixer, hidden, plain_fn, lengths=(223, 9), plan=((7, 0), (1, 4), (2, 1), (0, 1), (150, 3), (63, 0)),
                    loud_row=None):
    """A mixer with a fixed-size state, cut into steps (down to one row, up to 150), two requests side by side in
    slots 2 and 0; against the plain mixer on each whole sequence.  ``loud_row``: that row of request a is twelve
    times as large as the others, so that what it leaves in the state outweighs everything else for as long as the
    decays allow."""
    dtype = rt.dtype
    state = torch.zeros(3, mixer.cache_need().numel, device="cuda")
    view = StateView(state)
    g = torch.Generator().manual_seed(3)
    ha, hb = (torch.randn(n, hidden, generator=g) for n in lengths)
    if loud_row is not None:
        ha[loud_row] *= 12.0
    ha, hb = ha.to(dtype), hb.to(dtype)
    want_a, want_b = plain_fn(ha.double(), torch.arange(lengths[0])).float(), plain_fn(hb.double(), torch.arange(lengths[1])).float()
    got_a, got_b = [], []
    at = {2: 0, 0: 0}
    for na, nb in plan:
        ctx = step_ctx(rt, [(2, na), (0, nb)], at)
        rows = torch.cat([ha[at[2]:at[2] + na], hb[at[0]:at[0] + nb]]).cuda()
        out = dense_delta(ctx, mixer.forward(ctx, rows, view, True), dtype).float().cpu()
        got_a.append(out[:na]); got_b.append(out[na:na + nb])
        at[2] += na; at[0] += nb
    close(torch.cat(got_a), want_a, dtype, "request a")
    close(torch.cat(got_b), want_b, dtype, "request b")
    assert float(state[1].abs().max()) == 0.0          # nobody's slot


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,heads,dk,dv,rot", [(48, 2, 16, 8, 16), (40, 3, 10, 6, 4), (64, 1, 32, 64, 0), (96, 4, 64, 32, 32)])
def test_retention_alone(dtype, hidden, heads, dk, dv, rot):
    rt = Runtime(torch.device("cuda"), dtype)
    decay = [1.0 - 2.0 ** -(2 + h) for h in range(heads)]
    m = {"heads": heads, "dim": dk, "vdim": dv, "decay": decay, "rot": {"dims": rot, "base": 300.0}}
    mixer = build_part("mixer", PartSpec("retention", {"hidden": hidden, "n_heads": heads, "key_dim": dk, "value_dim": dv,
                                                       "decay": tuple(decay), "eps": 1e-5,
                                                       "position": PartSpec("rope", {"theta": 300.0, "dims": rot})}), rt)
    w = {k: v.double() for k, v in named(fill(mixer, 11, 0.4)).items()}
    run_state_mixer(rt, mixer, hidden, lambda h, pos: plain.mixer_retention(h, w, "p", m, 1e-5, pos))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,heads,d,rank", [(48, 2, 16, 8), (40, 5, 8, 4), (36, 3, 12, 5), (128, 2, 64, 24)])
def test_wkv_alone(dtype, hidden, heads, d, rank):
    """Token shift across the cuts (the row before a step's first row comes from the state), decays per channel,
    the bonus for the token itself."""
    rt = Runtime(torch.device("cuda"), dtype)
    m = {"heads": heads, "dim": d}
    mixer = build_part("mixer", PartSpec("wkv", {"hidden": hidden, "n_heads": heads, "head_dim": d, "decay_rank": rank, "eps": 1e-5}), rt)
    w = fill(mixer, 12, 0.4)
    for s in "rkvgw":                                   # blends between a row and the row before it
        w[f"mu.{s}"] = (0.5 + 0.3 * torch.randn(hidden, generator=torch.Generator().manual_seed(ord(s)))).to(torch.bfloat16).float()
    mixer.mu.copy_(torch.stack([w[f"mu.{s}"] for s in "rkvgw"]))
    w = {k: v.double() for k, v in named(w).items()}
    run_state_mixer(rt, mixer, hidden, lambda h, pos: plain.mixer_wkv(h, w, "p", m, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,heads,dk,dv,cap", [(48, 3, 16, 24, 6.0), (40, 1, 8, 40, 3.0), (36, 3, 5, 7, 2.0), (64, 2, 32, 32, 15.0)])
def test_mlstm_alone(dtype, hidden, heads, dk, dv, cap):
    """Gates whose exponentials only stay in range through the running maximum (large biases), the normaliser, the
    floor e^-m of the denominator."""
    rt = Runtime(torch.device("cuda"), dtype)
    m = {"heads": heads, "dim": dk, "vdim": dv, "gate_cap": cap}
    mixer = build_part("mixer", PartSpec("mlstm", {"hidden": hidden, "n_heads": heads, "key_dim": dk, "value_dim": dv,
                                                   "gate_cap": cap, "eps": 1e-5}), rt)
    w = fill(mixer, 13, 0.4)
    w["i.b"] = torch.linspace(-2.0, 3.0, heads)
    w["f.b"] = torch.linspace(4.0, 1.0, heads)
    mixer.b_gates.copy_(torch.cat([w["i.b"], w["f.b"]]))
    w = {k: v.double() for k, v in named(w).items()}
    run_state_mixer(rt, mixer, hidden, lambda h, pos: plain.mixer_mlstm(h, w, "p", m, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["retention", "wkv", "mlstm"])
@pytest.mark.parametrize("loud_row", [0, 3, 149])
def test_one_token_far_back_outweighs_the_rest(dtype, kind, loud_row):
    """Decays close to 1 and one loud token: hundreds of tokens later the outputs still consist mostly of what that
    token left in the state (the plain outputs with and without it differ by their whole size), through cuts into
    steps of 1 to 150 tokens.  A state that is lost, zeroed or taken from another slot on the way shows at once."""
    rt = Runtime(torch.device("cuda"), dtype)
    hidden, heads, dk, dv = 48, 2, 16, 16
    if kind == "retention":
        m = {"heads": heads, "dim": dk, "vdim": dv, "decay": [1.0, 0.9995], "rot": {"dims": 8, "base": 40.0}}
        mixer = build_part("mixer", PartSpec("retention", {"hidden": hidden, "n_heads": heads, "key_dim": dk, "value_dim": dv,
                                                           "decay": (1.0, 0.9995), "eps": 1e-5,
                                                           "position": PartSpec("rope", {"theta": 40.0, "dims": 8})}), rt)
        w = fill(mixer, 21, 0.3)
        fn = lambda wd: (lambda h, pos: plain.mixer_retention(h, wd, "p", m, 1e-5, pos))     # noqa: E731
    elif kind == "wkv":
        m = {"heads": heads, "dim": dk}
        mixer = build_part("mixer", PartSpec("wkv", {"hidden": hidden, "n_heads": heads, "head_dim": dk, "decay_rank": 8, "eps": 1e-5}), rt)
        w = fill(mixer, 22, 0.3)
        w["w0"] = torch.full_like(w["w0"], -7.0)            # decays of exp(-exp(-7 + small)): about 0.999 per token
        mixer.w_0.copy_(w["w0"])
        fn = lambda wd: (lambda h, pos: plain.mixer_wkv(h, wd, "p", m, 1e-5))     # noqa: E731
    else:
        m = {"heads": heads, "dim": dk, "vdim": dv, "gate_cap": 10.0}
        mixer = build_part("mixer", PartSpec("mlstm", {"hidden": hidden, "n_heads": heads, "key_dim": dk, "value_dim": dv,
                                                       "gate_cap": 10.0, "eps": 1e-5}), rt)
        w = fill(mixer, 23, 0.3)
        w["f.b"] = torch.full_like(w["f.b"], 8.0)           # forget gates of about 1 - e^-8
        mixer.b_gates[heads:].copy_(w["f.b"])
        fn = lambda wd: (lambda h, pos: plain.mixer_mlstm(h, wd, "p", m, 1e-5))     # noqa: E731
    wd = {k: v.double() for k, v in named(w).items()}
    run_state_mixer(rt, mixer, hidden, fn(wd), loud_row=loud_row)


WINDOW_SHAPES = [  # hidden, heads, kv heads, key size, value size, rotated dims, page, window
    (48, 4, 2, 16, 32, 8, 8, 9), (40, 3, 1, 24, 24, 0, 4, 5), (36, 5, 5, 12, 20, 12, 2, 3), (64, 6, 3, 40, 72, 20, 16, 100),
    (128, 8, 2, 64, 64, 64, 16, 40), (128, 4, 4, 32, 32, 16, 16, None), (64, 2, 1, 16, 16, 16, 8, 17), (64, 4, 2, 32, 16, 32, 8, 33),
]


def window_mixer(rt, shape, scale=None):
    hidden, heads, kv, dk, dv, rot, page, window = shape
    scale = scale or 1.5 / dk ** 0.5
    names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}
    spec = PartSpec("gqa_attention", {"hidden": hidden, "n_heads": heads, "n_kv_heads": kv, "head_dim": dk, "v_head_dim": dv,
                                      "qkv_bias": True, "scale": scale, "window": window, "names": names,
                                      "position": PartSpec("rope", {"theta": 500.0, "dims": rot})})
    m = {"heads": heads, "kv_heads": kv, "dim": dk, "vdim": dv, "scale": scale, "rot": {"dims": rot, "base": 500.0}}
    if window:
        m["mask"] = {"size": window}
    return build_part("mixer", spec, rt), m


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", WINDOW_SHAPES)
def test_window_attention_alone(dtype, shape):
    """Portions and single tokens of two requests side by side, whose earlier keys earlier calls wrote; windows
    shorter and longer than a page; keys and values of equal and of different sizes."""
    hidden, page, window = shape[0], shape[6], shape[7]
    rt = Runtime(torch.device("cuda"), dtype)
    mixer, m = window_mixer(rt, shape)
    w = {k: v.double() for k, v in named(fill(mixer, 6, 1.2 / hidden ** 0.5)).items()}     # scores of a few units
    cache = tw.CacheManager([(mixer.cache_need(), None)], page, 400 // page, 2, 400, dtype, rt.device, prefix_cache=False)
    a, b = cache.admit(None), cache.admit(None)
    g = torch.Generator().manual_seed(7)
    la, lb = 190, 60
    ha, hb = torch.randn(la, hidden, generator=g).to(dtype), torch.randn(lb, hidden, generator=g).to(dtype)
    want = {a.slot: plain.mixer_softmax(ha.double(), w, "p", m, torch.arange(la)).float(),
            b.slot: plain.mixer_softmax(hb.double(), w, "p", m, torch.arange(lb)).float()}
    rows_of = {a.slot: ha, b.slot: hb}
    at = {a.slot: 0, b.slot: 0}
    got = {a.slot: [], b.slot: []}
    for na, nb in [(0, 19), (13, 1), (150, 0), (1, 1), (1, 38), (2, 1), (1, 0), (22, 0)]:
        plan = [(a.slot, na), (b.slot, nb)]
        for lease, n in ((a, na), (b, nb)):
            cache.ensure(lease, at[lease.slot] + n)
        cache.sync_tables()
        ctx = step_ctx(rt, plan, at)
        rows = torch.cat([rows_of[s][at[s]:at[s] + n] for s, n in plan]).cuda()
        out = dense_delta(ctx, mixer.forward(ctx, rows, cache.view(0), True), dtype).float().cpu()
        assert int(ctx.status) == 0
        got[a.slot].append(out[:na]); got[b.slot].append(out[na:na + nb])
        for lease, n in ((a, na), (b, nb)):
            at[lease.slot] += n
            cache.advance(lease, None, at[lease.slot])
    for s in (a.slot, b.slot):
        close(torch.cat(got[s]), want[s], dtype, f"slot {s}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(48, 2, 1, 16, 32, 8, 8, 21), (64, 2, 2, 32, 32, 32, 16, 33), (40, 1, 1, 24, 8, 0, 4, 6)])
def test_one_key_at_the_window_edge(dtype, shape):
    """One key answers the last token's query far above all others, and its value stands out.  The key sits just
    inside the window, just outside, at page borders and at the first tokens; the asking token comes in a portion
    and alone.  An edge that is one token off changes the output by its whole size."""
    hidden, heads, kv, dk, dv, rot, page, window = shape
    rt = Runtime(torch.device("cuda"), dtype)
    mixer, m = window_mixer(rt, (hidden, heads, kv, dk, dv, 0, page, window), scale=6.4 / dk)     # no rotation: the match holds at any distance
    w = fill(mixer, 8, 0.02)
    g = torch.Generator().manual_seed(1)
    length = 4 * window + 7
    # queries and keys read channel 0 alone, strongly: a marked row (+1 there) meets a marked row with a score of
    # +6.4 and an unmarked row (-1) with -6.4; the values read channel 1, where only the marked key carries something
    w["q"][:, 0] = 1.0; w["k"][:, 0] = 1.0; w["v"][:, 0] = 0.0; w["v"][:, 1] = 2.0
    mixer.w_qkv[:, 0] = 1.0
    mixer.w_qkv[heads * dk + kv * dk:, 0] = 0.0
    mixer.w_qkv[heads * dk + kv * dk:, 1] = 2.0
    wd = {k: v.double() for k, v in named(w).items()}
    t = length - 1
    for j in [t - window + 1, t - window, t - window + 2, t - 1, 0, 1, page - 1, page, (t - window + 1) // page * page]:
        h = 0.1 * torch.randn(length, hidden, generator=g)
        h[:, 0] = -1.0
        h[:, 1] = 0.0
        h[j, 0], h[j, 1] = 1.0, 5.0
        h[t, 0] = 1.0
        h = h.to(dtype)
        want = plain.mixer_softmax(h.double(), wd, "p", m, torch.arange(length)).float()
        for tail in (0, 1, 9):                           # the asking token inside a portion, alone, after single tokens
            cache = tw.CacheManager([(mixer.cache_need(), None)], page, -(-length // page) + 1, 1, length + page, dtype, rt.device,
                                    prefix_cache=False, poison_freed=True)
            lease = cache.admit(None)
            at = {lease.slot: 0}
            outs = []
            for n in ([length] if tail == 0 else [length - tail] + [1] * tail):
                cache.ensure(lease, at[lease.slot] + n)
                cache.sync_tables()
                ctx = step_ctx(rt, [(lease.slot, n)], at)
                rows = h[at[lease.slot]:at[lease.slot] + n].cuda()
                outs.append(dense_delta(ctx, mixer.forward(ctx, rows, cache.view(0), True), dtype).float().cpu().clone())
                assert int(ctx.status) == 0
                at[lease.slot] += n
                cache.advance(lease, None, at[lease.slot])
            close(torch.cat(outs)[-1:], want[-1:], dtype, f"key at {j} (edge at {t - window + 1}), last {tail} tokens alone", bf16=0.1)
        seen = 0 <= t - j < window
        assert (float(want[-1].abs().max()) > 0.5) == seen, "the crafted key does not show in the plain output"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,experts,top,ff,shared", [(64, 6, 2, 40, 24), (40, 3, 1, 20, None), (36, 5, 5, 9, 27), (128, 10, 3, 88, 104)])
def test_routed_experts_alone(dtype, hidden, experts, top, ff, shared):
    """Router logits that stand apart (no close calls), the softmax over the chosen logits alone, the weighted sum,
    the shared expert behind its own gate."""
    rt = Runtime(torch.device("cuda"), dtype)
    spec = PartSpec("routed_experts", {"hidden": hidden, "experts": experts, "top": top, "intermediate": ff,
                                       "shared": PartSpec("swiglu", {"hidden": hidden, "intermediate": shared, "names": ("gate", "up", "down")}) if shared else None,
                                       "shared_gate": bool(shared)})
    part = build_part("feed_forward", spec, rt)
    w = fill(part, 14, 0.3)
    g = torch.Generator().manual_seed(2)
    rows = 37
    h = torch.randn(rows, hidden, generator=g).to(dtype)
    # logits spread over tens of units: rounding moves them by far less than the gaps between most of them
    w["router"] = (torch.randn(experts, hidden, generator=g) * 3).to(torch.bfloat16).float()
    w["router.b"] = torch.randn(experts, generator=g).to(torch.bfloat16).float()
    part.w_router.copy_(w["router"]); part.b_router.copy_(w["router.b"])
    wd = {k: v.double() for k, v in named(w).items()}
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.feed_forward_moe(h.double(), wd, "p", mlp).float()
    chosen_want, weight_want = plain.route(h.double(), wd, "p", top)
    ctx = ctx_of(rt, list(range(rows)), [0] * rows, [0], [0], [rows], [rows])
    chosen, weight, _ = part.route(ctx, h.cuda())
    margin = (h.double() @ wd["p.router"].T + wd["p.router.b"]).sort(dim=-1).values.diff(dim=-1).min(dim=-1).values
    sure = margin > 0.3
    assert int(sure.sum()) >= rows // 2
    assert torch.equal(chosen.cpu().long()[sure], chosen_want[sure])
    close(weight.cpu()[sure], weight_want[sure].float(), torch.float32, "weights of the chosen", f32=2e-2 if dtype == torch.bfloat16 else 1e-5)
    got = dense_delta(ctx, part.forward(ctx, h.cuda()), dtype).float().cpu()
    close(got[sure], want[sure], dtype, "routed feed-forward")


@pytest.mark.parametrize("dtype", DTYPES)
def test_weighted_sum_of_two_mixers(dtype):
    """Two mixers on the same rows, each with its own cache or state, summed with two scales."""
    rt = Runtime(torch.device("cuda"), dtype)
    hidden = 48
    cfg = parallel(left(4, 2, 16, 32, 9, 8, 1000.0, 0.3), right(3, 16, 24, 6.0), 0.7, -1.4)["mixer"]
    from tessweave_engine_b200.config.sapatar_config import ParallelConfig, SapatarConfig
    from tessweave_engine_b200.models.sapatar import mixer_spec
    typed = SapatarConfig.from_dict({"vocab": 8, "width": hidden, "norm": {"eps": 1e-5},
                                     "layers": [{"type": "parallel", "mixer": cfg, "mlp": None}]})
    mixer = build_part("mixer", mixer_spec(typed, typed.layers[0], "layer"), rt)
    w = {k: v.double() for k, v in named(fill(mixer, 5, 0.3)).items()}
    cache = tw.CacheManager([(mixer.cache_need(), None)], 8, 16, 2, 96, dtype, rt.device, prefix_cache=False)
    assert isinstance(cache.view(0), SeveralViews)
    lease = cache.admit(None)
    h = torch.randn(50, hidden, generator=torch.Generator().manual_seed(9)).to(dtype)
    want = plain.mixer("parallel", h.double(), w, "p", cfg, 1e-5, torch.arange(50)).float()
    at, outs = {lease.slot: 0}, []
    for n in (20, 1, 1, 28):
        cache.ensure(lease, at[lease.slot] + n)
        cache.sync_tables()
        ctx = step_ctx(rt, [(lease.slot, n)], at)
        outs.append(dense_delta(ctx, mixer.forward(ctx, h[at[lease.slot]:at[lease.slot] + n].cuda(), cache.view(0), True), dtype).float().cpu().clone())
        at[lease.slot] += n
        cache.advance(lease, None, at[lease.slot])
    close(torch.cat(outs), want, dtype, "left and right")


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------
def settle_router(folder):
    """For bfloat16 runs: a router whose choice no rounding can turn.  The biases stand 3 apart in an order of the
    layer's own and the matrix moves a logit by a fraction of that, so every token of a layer chooses the same
    experts, with weights that still depend on the token.  (The choice per token is what the float32 runs, whose
    routers are as random as every other matrix, and the test of the part alone check.)"""
    from safetensors.torch import load_file, save_file
    t = load_file(str(folder / "model.safetensors"))
    for name in sorted(t):
        if name.endswith(".mlp.router"):
            g = torch.Generator().manual_seed(len(name) + t[name].shape[0])
            t[name] = (t[name].float() * 0.2).to(t[name].dtype)
            t[name + ".b"] = (torch.randperm(t[name].shape[0], generator=g).float() * 3.0).to(t[name + ".b"].dtype)
    save_file(t, str(folder / "model.safetensors"), metadata={"format": "pt"})
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(name, dtype) -> model folder.  The bfloat16 runs get a copy whose routers are settled and whose norms have a
    large eps: a head's state after a request's first token has rank one, so its output is (q . k) v, and the norm over
    the head turns that into sign(q . k) times a unit vector unless eps is felt; with the tiny eps of the float32
    models a rounding of q or k that turns the sign of a nearly orthogonal pair moves the row, and the rows behind it,
    by tens of per cent.  (The float32 runs, which no rounding turns, keep the tiny eps.)"""
    tmp = tmp_path_factory.mktemp("sapatar")
    out = {}
    for name, cfg in SAPATAR_CONFIGS.items():
        out[name, "float32"] = tw.write_random_model(tmp / name, cfg, seed=SAPATAR_SEEDS[name], std=SAPATAR_STD[name])
        out[name, "bfloat16"] = settle_router(tw.write_random_model(tmp / f"{name}_settled", {**cfg, "norm": {"eps": 0.05}},
                                                                    seed=SAPATAR_SEEDS[name], std=SAPATAR_STD[name]))
    return out


LENGTHS = [70, 1, 45, 100, 2, 33, 64, 129]


def requests_for(name):
    return {f"r{i}": random_tokens(SAPATAR_CONFIGS[name]["vocab"], n, 20 + i) for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def plain_rows(folders):
    return {key: {rid: plain.logits_of(folder, t).numpy() for rid, t in requests_for(key[0]).items()}
            for key, folder in folders.items()}


def row_error(row, ref):
    d = row - ref
    return float(np.sqrt(np.mean((d - d.mean()) ** 2)) / max(np.sqrt(np.mean((ref - ref.mean()) ** 2)), 1e-6))


@pytest.fixture(scope="module")
def float32_noise(folders, plain_rows):
    """What 32-bit arithmetic alone does to each row: the plain implementation in float32 against itself in float64.
    (Model A has rows where that is 3e-4 of the row's spread: a denominator near its floor; most rows are near 1e-6.)"""
    out = {}
    for name in SAPATAR_CONFIGS:
        for rid, t in requests_for(name).items():
            low = plain.logits_of(folders[name, "float32"], t, torch.float32).numpy()
            out[name, rid] = [row_error(low[p], plain_rows[name, "float32"][rid][p]) for p in range(len(t))]
    return out


@pytest.fixture(scope="module")
def bfloat16_noise(folders, plain_rows):
    """What perturbations of bfloat16's size do to each row by themselves: the plain implementation (float64) with
    every matrix element moved by a relative 2^-8 times a normal draw, against itself.  Rows behind a nearly
    orthogonal query and key at a request's first tokens, or near a denominator's floor, move by tens of per cent."""
    out = {}
    for name in SAPATAR_CONFIGS:
        config, weights = plain.read_folder(folders[name, "bfloat16"], torch.float64)
        g = torch.Generator().manual_seed(99)
        moved = {k: v * (1 + 2.0 ** -8 * torch.randn(v.shape, generator=g, dtype=torch.float64)) if v.dim() == 2 else v
                 for k, v in weights.items()}
        for rid, t in requests_for(name).items():
            low = plain.forward(config, moved, t).float().numpy()
            out[name, rid] = [row_error(low[p], plain_rows[name, "bfloat16"][rid][p]) for p in range(len(t))]
    return out


def compare(rows, want, dtype, what, noise=None):
    """Every logits row against the plain one (float64).  float32: every row within 5e-5 of its spread plus four
    times what the plain implementation loses at that row when it runs in float32 itself.  bfloat16: the design has
    places where rounding alone moves a row far (under the matrix memory's normaliser the sign of a nearly orthogonal
    query and key decides a head's output at a request's first tokens), so the rows are judged together: the median
    within 6 % (observed: 1 to 4.4 %), at most five rows in a hundred beyond 8 % plus three times what a perturbation
    of bfloat16's size does to that row of the plain implementation (``noise``), none that is not finite.  A lost
    state, a key outside its window or a wrong page moves rows by their whole size."""
    errors, over = [], []
    for (rid, p), row in rows.items():
        err = row_error(row, want[rid][p])
        assert np.isfinite(row).all(), f"{what}: {rid}[{p}] is not finite"
        lost = noise[rid][p] if noise else 0.0
        if dtype == "float32":
            assert err <= 5e-5 + 4 * lost, f"{what}: {rid}[{p}] differs by {err:.3g} of the row's spread (float32 alone: {lost:.3g})"
        elif err > 8e-2 + 3 * lost:
            over.append((rid, p, round(err, 3)))
        errors.append(err)
    if dtype == "bfloat16":
        assert float(np.median(errors)) <= 6e-2, f"{what}: the median row differs by {float(np.median(errors)):.3g}"
        assert len(over) <= max(2, 5 * len(errors) // 100), f"{what}: {len(over)} of {len(errors)} rows are far off: {over[:8]}"


SCHEDULES = {
    "whole": schedule_whole,
    "tail": schedule_tail,
    "portions": schedule_portions,
    "one_by_one": lambda r: schedule_portions({k: v for k, v in r.items() if len(v) <= 70}, sizes=(1,)),
    "mixed": lambda r: schedule_mixed(r, live=4, seed=1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cutting_gives_the_plain_logits(name, dtype, folders, plain_rows, float32_noise, bfloat16_noise, tmp_path):
    """Whole prompts; most of a prompt and its last 32 tokens one by one; portions down to two tokens; token by
    token from the first; four live requests in mixed batches with so few pages and slots that both are used
    again (freed pages are filled with NaN first)."""
    reqs = requests_for(name)
    for kind, make in SCHEDULES.items():
        steps = make(reqs)
        rows = replay_in_process(folders[name, dtype], dtype, steps, tmp_path / kind, block_size=SAPATAR_PAGE[name],
                                 max_tokens=max_live_tokens(steps))
        assert rows, kind
        noise = float32_noise if dtype == "float32" else bfloat16_noise
        compare(rows, plain_rows[name, dtype], dtype, f"{name} {kind}", {rid: noise[name, rid] for rid in reqs})


def test_batches_and_cuts_do_not_change_a_request(folders, tmp_path):
    """float32: a request's logits in a mixed batch, or cut into portions, equal those it gets alone, to rounding."""
    reqs = requests_for("B")
    folder = folders["B", "float32"]
    alone = replay_in_process(folder, "float32", schedule_whole(reqs), tmp_path / "alone", block_size=4)
    for kind, steps in (("mixed", schedule_mixed(reqs, live=4, seed=3)), ("portions", schedule_portions(reqs))):
        got = replay_in_process(folder, "float32", steps, tmp_path / kind, block_size=4)
        worst = max(float(np.abs(row - alone[key]).max() / np.abs(alone[key]).max()) for key, row in got.items())
        assert worst <= 1e-4, (kind, worst)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(dtype, folders, tmp_path):
    """A short prompt and 300 tokens one by one: the windows pass over decoded tokens only, pages of the windowed
    layers are given back and used again on the way, the states carry everything else."""
    name = "C"
    toks = random_tokens(SAPATAR_CONFIGS[name]["vocab"], 310, 77)
    steps = schedule_tail({"long": toks}, tail=300)
    rows = replay_in_process(folders[name, dtype], dtype, steps, tmp_path / "out", block_size=SAPATAR_PAGE[name], max_tokens=384)
    want = plain.logits_of(folders[name, dtype], toks).numpy()
    low = plain.logits_of(folders[name, dtype], toks, torch.float32).numpy()
    compare(rows, {"long": want}, dtype, "long decoding", {"long": [row_error(low[p], want[p]) for p in range(len(toks))]})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_hundreds_of_tokens_past_windows_of_tensor_core_sizes(dtype, tmp_path):
    """Keys and values of one size (64, 32), windows of 70 and 150, prompts of 420 and 190 tokens: whole, with the last
    40 tokens one by one, and in mixed batches, on pages of 16 that the windows give back on the way."""
    cfg = SAPATAR_E if dtype == "float32" else {**SAPATAR_E, "norm": {"eps": 0.05}}
    folder = tw.write_random_model(tmp_path / "model", cfg, seed=31, std=0.1)
    if dtype == "bfloat16":
        settle_router(folder)
    reqs = {"long": random_tokens(cfg["vocab"], 420, 5), "mid": random_tokens(cfg["vocab"], 190, 6), "short": random_tokens(cfg["vocab"], 37, 7)}
    want = {rid: plain.logits_of(folder, t).numpy() for rid, t in reqs.items()}
    if dtype == "float32":
        noise = {rid: [row_error(r, w) for r, w in zip(plain.logits_of(folder, t, torch.float32).numpy(), want[rid])] for rid, t in reqs.items()}
    else:
        config, weights = plain.read_folder(folder, torch.float64)
        g = torch.Generator().manual_seed(98)
        moved = {k: v * (1 + 2.0 ** -8 * torch.randn(v.shape, generator=g, dtype=torch.float64)) if v.dim() == 2 else v
                 for k, v in weights.items()}
        noise = {rid: [row_error(r, w) for r, w in zip(plain.forward(config, moved, t).float().numpy(), want[rid])] for rid, t in reqs.items()}
    for kind, steps in (("whole", schedule_whole(reqs)), ("tail", schedule_tail(reqs, tail=40)),
                        ("mixed", schedule_mixed(reqs, live=3, seed=2, prefill=(33, 2, 70, 5, 128, 16)))):
        rows = replay_in_process(folder, dtype, steps, tmp_path / kind, block_size=16, max_tokens=max_live_tokens(steps))
        compare(rows, want, dtype, f"E {kind}", noise)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(name, dtype, folders):
    """``generate`` (scheduler, continuous batching, CUDA graphs, look-ahead) against the plain greedy loop;
    every chosen token must be the plain implementation's best on that path, or nearly."""
    prompts = [random_tokens(SAPATAR_CONFIGS[name]["vocab"], n, 60 + n) for n in (21, 5, 40)]
    model = tw.load_model(folders[name, dtype], dtype, "cuda")
    out = tw.generate(model, prompts, max_tokens=12, ignore_eos=True,
                      engine_config=tw.EngineConfig(block_size=SAPATAR_PAGE[name], kv_blocks=40, max_context=128, max_active=2,
                                                    prefill_chunk=16))
    config, weights = plain.read_folder(folders[name, dtype], torch.float64)
    for p, o in zip(prompts, out):
        assert len(o) == 12
        logits = plain.forward(config, weights, p + o).float()
        for i, t in enumerate(o):
            row = logits[len(p) + i - 1]
            gap = float(row.max() - row[t])
            spread = float(row.std())
            assert gap <= (1e-4 if dtype == "float32" else 0.15) * spread, f"token {i} lies {gap:.3g} below the best (spread {spread:.3g})"
