"""The Linurax decoder in the engine against the plain implementation (tests/plain_linurax.py): every
mechanism alone, then whole models under every way of cutting and batching the work, in float32 and
bfloat16.  The tiny models and their weights are made here."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_linurax as plain
from helpers import (max_live_tokens, random_tokens, replay_in_process, schedule_mixed, schedule_portions, schedule_tail,
                     schedule_whole)
from tiny_linurax import LINURAX_CONFIGS, LINURAX_PAGE, LINURAX_SEEDS, LINURAX_STD, attention, mingru

import tessweave_engine_b200 as tw
from tessweave_engine_b200.csrc import ops
from tessweave_engine_b200.engine.runner import ModelRunner, StepEntry
from tessweave_engine_b200.parts import PartSpec, Runtime, StepContext, Workspace, build_part, dense_delta

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def ctx_of(rt, positions, seq_of_token, slots, q_start, q_len, kv_len):
    """A StepContext as the runner would stage it, for running one part outside a model."""
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")     # noqa: E731
    n = len(positions)
    return StepContext(runtime=rt, workspace=Workspace(torch.device("cuda")), n_tokens=n, n_seqs=len(slots),
                       token_ids=i32([0] * n), positions=i32(positions), seq_of_token=i32(seq_of_token),
                       seq_slot=i32(slots), seq_q_start=i32(q_start), seq_q_len=i32(q_len), seq_kv_len=i32(kv_len),
                       status=torch.zeros(1, dtype=torch.int32, device="cuda"), host_slot=slots, host_q_start=q_start,
                       host_q_len=q_len, host_kv_len=kv_len, max_q_len=max(q_len), max_kv_len=max(kv_len),
                       decode_only=all(c == 1 for c in q_len))


def fill(part, seed, std):
    """Random weights straight into a part; returns them by name as fp32 CPU tensors (bf16 values in bf16 runs)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for decl in part.weights():
        t = torch.randn(decl.shape, generator=g) * std
        if decl.init == "one_plus_normal":
            t = 1 + 0.1 * t / std
        if decl.init == "eye_plus_normal":
            t = torch.eye(decl.shape[0]) + t
        t = t.to(torch.bfloat16).float()          # exact in both run types
        decl.dest.copy_(t.view(decl.dest.shape))
        out[decl.name] = t
    return out


def close(got, want, dtype, what, f32=2e-5, bf16=3e-2):
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    bound = (f32 if dtype == torch.float32 else bf16) * max(scale, 1e-6)
    assert err <= bound, f"{what}: differs by {err:.3g} (scale {scale:.3g}, bound {bound:.3g})"


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,dims,theta", [(16, 8, 1e3), (24, 24, 5e4), (64, 2, 1e6), (32, 0, 1e4)])
def test_interleaved_rotation_alone(dtype, head_dim, dims, theta):
    """Neighbouring pairs of the first ``dims`` values rotate; the rest of a head and the heads behind stay."""
    rt = Runtime(torch.device("cuda"), dtype)
    rope = build_part("position", PartSpec("rope_interleaved", {"theta": theta, "dims": dims}), rt)
    positions = [0, 1, 2, 700, 3, 15, 16, 4095]
    ctx = ctx_of(rt, positions, [0, 0, 0, 1, 2, 2, 2, 3], [0, 1, 2, 3], [0, 3, 4, 7], [3, 1, 3, 1], [3, 701, 17, 4096])
    heads, extra = 5, 2
    x = torch.randn(len(positions), (heads + extra) * head_dim, generator=torch.Generator().manual_seed(4)).to(dtype)
    qk = x.cuda().clone()
    rope.apply(ctx, qk, heads, head_dim)
    ref = x.float().reshape(len(positions), heads + extra, head_dim)
    want = plain.rotate_interleaved(ref[:, :heads], torch.tensor(positions), dims, theta) if dims else ref[:, :heads]
    got = qk.float().cpu().reshape(len(positions), heads + extra, head_dim)
    close(got[:, :heads], want, dtype, "rotation")
    assert torch.equal(got[:, heads:], ref[:, heads:])
    assert torch.equal(got[:, :heads, dims:], ref[:, :heads, dims:])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [40, 64, 1000, 9000])
def test_norm_of_a_sublayer_output_into_the_stream(dtype, hidden):
    """resid += rms(delta) * w in fp32, for a tensor and for the slices of a split product; the copy in the
    run's type is the rounded new stream."""
    rt = Runtime(torch.device("cuda"), dtype)
    norm = build_part("norm", PartSpec("rmsnorm", {"size": hidden, "eps": 1e-5, "weight_name": ""}), rt)
    assert [d.name for d in norm.weights()] == [""]
    g = torch.Generator().manual_seed(hidden)
    w = (1 + 0.2 * torch.randn(hidden, generator=g))
    norm.weight.copy_(w)
    rows = 5
    resid0 = torch.randn(rows, hidden, generator=g) * 3
    delta = (torch.randn(rows, hidden, generator=g) * 40).to(dtype)
    want = resid0 + plain.rms(delta.float(), w, 1e-5)
    ctx = ctx_of(rt, list(range(rows)), [0] * rows, [0], [0], [rows], [rows])
    for split in (False, True):
        resid = resid0.cuda().clone()
        copy = torch.full((rows, hidden), float("nan"), dtype=dtype, device="cuda")
        if split:
            parts = torch.randn(3, rows, hidden, generator=g)
            parts[2] = delta.float() - parts[0] - parts[1]
            src = ops.SplitSum(parts.cuda())
            ref = resid0 + plain.rms(parts[0] + parts[1] + parts[2], w, 1e-5)
        else:
            src, ref = delta.cuda(), want
        norm.add_normed(ctx, resid, src, rows, copy)
        close(resid.cpu(), ref, torch.float32, f"stream (split={split})", f32=3e-6)
        assert torch.equal(copy.cpu(), resid.cpu().to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding_and_tied_head(dtype):
    rt = Runtime(torch.device("cuda"), dtype)
    vocab, hidden = 131, 72
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab": vocab, "hidden": hidden, "scale": 7.25,
                                                              "weight_name": ""}), rt)
    assert [d.name for d in emb.weights()] == [""]
    emb.weight.copy_(torch.randn(vocab, hidden, generator=torch.Generator().manual_seed(8)))
    ids = [0, 130, 5, 5, 99]
    ctx = ctx_of(rt, [0, 1, 2, 3, 4], [0] * 5, [0], [0], [5], [5])
    ctx.token_ids = torch.tensor(ids, dtype=torch.int32, device="cuda")
    stream = emb.forward(ctx)
    assert torch.equal(stream.resid, emb.weight[ids].float() * 7.25)
    head = build_part("head", PartSpec("linear_head", {"vocab": vocab, "hidden": hidden}), rt, tied=emb.shared_matrix())
    y = (torch.randn(3, hidden, generator=torch.Generator().manual_seed(9)) * 0.5).to(dtype).cuda()
    logits = torch.zeros(3, vocab, device="cuda")
    head.forward(ctx, logits, y, 3)
    close(logits.cpu(), y.float().cpu() @ emb.weight.float().cpu().t(), dtype, "tied head reads the unscaled matrix", bf16=2e-3)


ATTENTION_SHAPES = [  # hidden, heads, kv heads, head size, rotated dims, page, window
    (48, 4, 2, 16, 8, 8, None), (40, 3, 1, 24, 24, 4, None), (64, 1, 1, 32, 0, 8, None), (96, 6, 6, 16, 16, 16, None),
    (128, 12, 2, 64, 32, 16, None), (128, 20, 4, 32, 16, 8, None), (48, 4, 2, 16, 8, 8, 11), (40, 3, 1, 24, 24, 4, 7),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_sigmoid_attention_alone(dtype, shape):
    """The mixer on hand-made rows: a portion of request a beside a single token of request b, whose earlier
    keys an earlier call wrote; then a's next portion.  Against the plain mixer on each whole sequence."""
    hidden, heads, kv, d, rot, page, window = shape
    rt = Runtime(torch.device("cuda"), dtype)
    spec = PartSpec("sigmoid_attention", {"hidden": hidden, "n_heads": heads, "n_kv_heads": kv, "head_dim": d,
                                          "scale": 1.5 / d ** 0.5, "eps": 1e-5, "window": window,
                                          "position": PartSpec("rope_interleaved", {"theta": 500.0, "dims": rot})})
    mixer = build_part("mixer", spec, rt)
    w = fill(mixer, 6, 0.3)
    w["pb"] = w["pb"] - 1.0
    mixer.bias.copy_(w["pb"])
    params = {"heads": heads, "kv_heads": kv, "dim": d, "scale": 1.5 / d ** 0.5, "rot": {"dims": rot, "base": 500.0}}
    cache = tw.CacheManager([(mixer.cache_need(), None)], page, 24, 2, 96, dtype, rt.device, prefix_cache=False)
    a, b = cache.admit(None), cache.admit(None)
    g = torch.Generator().manual_seed(7)
    ha, hb = (torch.randn(30, hidden, generator=g)).to(dtype), (torch.randn(20, hidden, generator=g)).to(dtype)
    want_a = plain.sigmoid_attention(ha.float(), w, params, 1e-5, window=window)
    want_b = plain.sigmoid_attention(hb.float(), w, params, 1e-5, window=window)

    def run(ctx, h):
        cache.sync_tables()
        out = dense_delta(ctx, mixer.forward(ctx, h.cuda(), cache.view(0), True), dtype).float().cpu()
        assert int(ctx.status) == 0
        return out

    cache.ensure(b, 19)
    got_b0 = run(ctx_of(rt, list(range(19)), [0] * 19, [b.slot], [0], [19], [19]), hb[:19])
    cache.ensure(a, 13); cache.ensure(b, 20)
    got = run(ctx_of(rt, list(range(13)) + [19], [0] * 13 + [1], [a.slot, b.slot], [0, 13], [13, 1], [13, 20]),
              torch.cat([ha[:13], hb[19:]]))
    cache.ensure(a, 30)
    got_a1 = run(ctx_of(rt, list(range(13, 30)), [0] * 17, [a.slot], [0], [17], [30]), ha[13:])
    close(got_b0, want_b[:19], dtype, "b's first portion")
    close(got[:13], want_a[:13], dtype, "a's first portion beside b")
    close(got[13:], want_b[19:], dtype, "b's single token beside a")
    close(got_a1, want_a[13:], dtype, "a's second portion")


@pytest.mark.parametrize("prefill", ["mma", "tcgen05"])
@pytest.mark.parametrize("heads,kv,d,window,page", [
    (8, 2, 64, None, 16), (20, 4, 32, None, 16), (3, 1, 96, None, 16), (4, 4, 128, 150, 16), (2, 1, 16, 65, 16), (28, 4, 128, None, 16),
    (6, 3, 64, 300, 16), (40, 8, 16, None, 8),          # more heads than one block of the single-token kernel serves
    (8, 2, 64, None, 128), (4, 2, 128, 200, 256),       # pages as long as a key tile, and longer
    (6, 3, 64, None, 4)])                               # 32 pages to a key tile
def test_tensor_core_attention_against_the_exact_kernel(heads, kv, d, window, page, prefill, monkeypatch):
    """bfloat16, several hundred keys: portions whose tiles end inside pages and inside tiles of 64 keys, and
    single tokens whose keys are cut into slices, through the tensor-core kernels and through the exact kernel
    (same rounded inputs, so they differ by the rounding of the weights to bfloat16 and no more).  Portions run
    on the mma.sync kernel and on the tcgen05 kernel."""
    hidden = 64
    if prefill == "tcgen05" and d not in (64, 128):
        pytest.skip("the tcgen05 kernel is built for head sizes 64 and 128")
    monkeypatch.setenv("TESSWEAVE_SIGMOID_PREFILL", prefill)     # tcgen05: every portion, also the short ones
    rt = Runtime(torch.device("cuda"), torch.bfloat16)
    spec = PartSpec("sigmoid_attention", {"hidden": hidden, "n_heads": heads, "n_kv_heads": kv, "head_dim": d,
                                          "scale": 1.2 / d ** 0.5, "eps": 1e-5, "window": window,
                                          "position": PartSpec("rope_interleaved", {"theta": 1e4, "dims": d // 2})})
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(700, hidden, generator=g).to(torch.bfloat16)
    cuts = [200, 1, 57, 130, 1, 1, 64, 1, 193, 1, 1, 50]
    results = {}
    for mode in ("tensor", "exact"):
        if mode == "exact":
            monkeypatch.setenv("TESSWEAVE_SIGMOID_ATTENTION", "exact")
        mixer = build_part("mixer", spec, rt)
        fill(mixer, 21, 0.3)
        mixer.bias.fill_(-2.0)
        cache = tw.CacheManager([(mixer.cache_need(), None)], page, -(-768 // page), 1, 768, torch.bfloat16, rt.device, prefix_cache=False)
        lease = cache.admit(None)
        outs, p = [], 0
        for n in cuts:
            cache.ensure(lease, p + n)
            cache.sync_tables()
            ctx = ctx_of(rt, list(range(p, p + n)), [0] * n, [lease.slot], [0], [n], [p + n])
            outs.append(mixer.attend(ctx, mixer.project_in(ctx, rows[p:p + n].cuda()), cache.view(0), True).float().cpu().clone())
            assert int(ctx.status) == 0
            p += n
        results[mode] = torch.cat(outs)
    scale = float(results["exact"].abs().max())
    assert float((results["tensor"] - results["exact"]).abs().max()) <= 0.02 * scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,width", [(48, 80), (40, 33), (128, 300)])
def test_mingru_alone(dtype, hidden, width):
    """The recurrence cut into steps (down to one row, up to 150), two requests side by side, the state carried in slots."""
    rt = Runtime(torch.device("cuda"), dtype)
    mixer = build_part("mixer", PartSpec("mingru", {"hidden": hidden, "width": width}), rt)
    w = fill(mixer, 11, 0.4)
    state = torch.zeros(3, width, device="cuda")
    view = tw.parts.StateView(state)
    g = torch.Generator().manual_seed(3)
    ha, hb = torch.randn(223, hidden, generator=g).to(dtype), torch.randn(9, hidden, generator=g).to(dtype)
    want_a, want_b = plain.mingru(ha.float(), w), plain.mingru(hb.float(), w)
    got_a, got_b = [], []
    # (rows of a, rows of b) per step; a sits in slot 2, b in slot 0
    # a portion of more than 64 rows is cut into segments that are chained inside the kernel
    plan = [(7, 0), (1, 4), (2, 1), (0, 1), (150, 3), (63, 0)]
    pa = pb = 0
    for na, nb in plan:
        rows = [ha[pa:pa + na], hb[pb:pb + nb]]
        slots, starts, lens, seq_of = [], [], [], []
        for i, (slot, n) in enumerate(((2, na), (0, nb))):
            if n:
                seq_of += [len(slots)] * n
                starts.append(sum(lens)); lens.append(n); slots.append(slot)
        ctx = ctx_of(rt, [0] * (na + nb), seq_of, slots, starts, lens, lens)
        out = dense_delta(ctx, mixer.forward(ctx, torch.cat(rows).cuda(), view, True), dtype).float().cpu()
        got_a.append(out[:na]); got_b.append(out[na:])
        pa, pb = pa + na, pb + nb
    close(torch.cat(got_a), want_a, dtype, "request a")
    close(torch.cat(got_b), want_b, dtype, "request b")
    assert float(state[1].abs().max()) == 0.0          # nobody's slot


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("linurax")
    return {name: tw.write_random_model(tmp / name, cfg, seed=LINURAX_SEEDS[name], std=LINURAX_STD[name])
            for name, cfg in LINURAX_CONFIGS.items()}


LENGTHS = [70, 1, 45, 100, 2, 33, 64, 129]


def requests_for(name):
    return {f"r{i}": random_tokens(LINURAX_CONFIGS[name]["vocab"], n, 20 + i) for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def plain_rows(folders):
    return {name: {rid: plain.logits_of(folders[name], t).numpy() for rid, t in requests_for(name).items()}
            for name in LINURAX_CONFIGS}


def compare(rows, want, dtype, what):
    """Every logits row against the plain one: 1e-5 of the logits' scale in float32, 4 % in bfloat16
    (mean taken off, as a constant shift of a row changes no choice)."""
    worst = 0.0
    for (rid, p), row in rows.items():
        ref = want[rid][p]
        d = row - ref
        err = float(np.sqrt(np.mean((d - d.mean()) ** 2)) / max(np.sqrt(np.mean((ref - ref.mean()) ** 2)), 1e-6))
        assert np.isfinite(row).all(), f"{what}: {rid}[{p}] is not finite"
        worst = max(worst, err)
        assert err <= (2e-5 if dtype == "float32" else 4e-2), f"{what}: {rid}[{p}] differs by {err:.3g} of the row's spread"
    return worst


SCHEDULES = {
    "whole": schedule_whole,
    "tail": schedule_tail,
    "portions": schedule_portions,
    "one_by_one": lambda r: schedule_portions({k: v for k, v in r.items() if len(v) <= 70}, sizes=(1,)),
    "mixed": lambda r: schedule_mixed(r, live=4, seed=1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cutting_gives_the_plain_logits(name, dtype, folders, plain_rows, tmp_path):
    """Whole prompts; most of a prompt and its last 32 tokens one by one; portions down to two tokens; token by
    token from the first; four live requests in mixed batches with so few pages and slots that both are used
    again (freed pages are filled with NaN first)."""
    reqs = requests_for(name)
    for kind, make in SCHEDULES.items():
        steps = make(reqs)
        rows = replay_in_process(folders[name], dtype, steps, tmp_path / kind, block_size=LINURAX_PAGE[name],
                                 max_tokens=max_live_tokens(steps))
        assert rows, kind
        compare(rows, plain_rows[name], dtype, f"{name} {kind}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_and_short_portions_and_single_tokens_in_one_step(dtype, folders, plain_rows, tmp_path):
    """One step carries a portion of 150 tokens (which the tcgen05 kernel takes in bfloat16), portions of 3 and 40, and
    single tokens of two requests with keys in the cache; the next step continues all of them."""
    name = "C"
    vocab = LINURAX_CONFIGS[name]["vocab"]
    reqs = {"long": random_tokens(vocab, 300, 90), "tiny": random_tokens(vocab, 9, 91), "mid": random_tokens(vocab, 90, 92),
            "one": random_tokens(vocab, 70, 93), "two": random_tokens(vocab, 131, 94)}
    plan = [{"one": 68, "two": 129}, {"long": 150, "tiny": 3, "mid": 40, "one": 1, "two": 1},
            {"long": 150, "tiny": 6, "mid": 50, "one": 1, "two": 1}]
    at = {k: 0 for k in reqs}
    steps = []
    for i, counts in enumerate(plan):
        entries = []
        for rid, n in counts.items():
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + n], "want": list(range(n))})
            at[rid] += n
        steps.append({"step": i, "entries": entries, "end": [rid for rid in counts if at[rid] == len(reqs[rid])]})
    assert all(at[k] == len(v) for k, v in reqs.items())
    rows = replay_in_process(folders[name], dtype, steps, tmp_path / "out", block_size=LINURAX_PAGE[name], max_tokens=1024)
    want = {rid: plain.logits_of(folders[name], toks).numpy() for rid, toks in reqs.items()}
    compare(rows, want, dtype, "long and short portions beside single tokens")


def test_batches_do_not_change_a_request(folders, tmp_path):
    """float32: a request's logits in a mixed batch equal those it gets alone, to rounding."""
    reqs = requests_for("A")
    alone = replay_in_process(folders["A"], "float32", schedule_whole(reqs), tmp_path / "alone", block_size=8)
    steps = schedule_mixed(reqs, live=4, seed=3)
    mixed = replay_in_process(folders["A"], "float32", steps, tmp_path / "mixed", block_size=8)
    for key, row in mixed.items():
        assert np.abs(row - alone[key]).max() <= 2e-5 * np.abs(alone[key]).max(), key


MATCH_QUERY, MATCH_KEY = 7, 11       # the token whose query finds the key of the other


def craft_match_model(tmp, page):
    """A model whose first layer's attention answers to ONE earlier key.  Head 0's query matrix is the key
    matrix with the two halves of a head's unrotated part swapped (R), and the embedding of token MATCH_KEY is
    chosen so that its key is R applied to the key of token MATCH_QUERY: the query of MATCH_QUERY meets that key
    with a score far above all others (and not its own key, nor an equal value: the values are the keys, so
    the matched value differs from the query token's own).  The heads are not mixed, the score's bias is far
    below zero and the scale is large: a key of another token weighs about e^-8, the matched key at least 1/2.
    A key that is lost, read from a wrong page or rotated by a wrong position changes the logits by much more
    than bfloat16 rounding does.  Only a quarter of a head is rotated, so the match survives any distance."""
    d, heads, rot, width = 32, 2, 8, 48
    cfg = {"architecture": "Linurax", "vocab": 120, "width": width, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
           "layers": [attention(heads, 1, d, rot, 100.0, 0.5), mingru(40, ff=56)]}
    folder = tw.write_random_model(Path(tmp) / f"match{page}", cfg, seed=9, std=0.3)
    from safetensors.torch import load_file, save_file
    t = load_file(str(folder / "model.safetensors"))
    wk = t["l0.mix.k"].float()
    half = (d - rot) // 2
    swap = list(range(rot)) + list(range(rot + half, d)) + list(range(rot, rot + half))
    t["l0.mix.q"][:d] = wk[swap].to(t["l0.mix.q"].dtype)
    embed = t["embed"].float()
    embed[MATCH_KEY] = torch.linalg.pinv(wk) @ (wk @ embed[MATCH_QUERY])[swap]
    t["embed"] = embed.to(t["embed"].dtype)
    t["l0.mix.q.norm"] = torch.ones_like(t["l0.mix.q.norm"])
    t["l0.mix.k.norm"] = torch.ones_like(t["l0.mix.k.norm"])
    t["l0.mix.talk"] = torch.eye(heads).to(t["l0.mix.talk"].dtype)
    t["l0.mix.pb"] = torch.full_like(t["l0.mix.pb"], -8.0)
    save_file(t, str(folder / "model.safetensors"), metadata={"format": "pt"})
    return folder, cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_key_far_back_at_every_kind_of_place(dtype, tmp_path):
    """The matched key at place j, the token that asks for it at the end.  j runs over the first tokens, both
    sides of page borders, and far back among hundreds; the last token comes in a prompt portion, alone after
    a portion, and after many single tokens."""
    page = 16
    folder, cfg = craft_match_model(tmp_path, page)
    length = 330
    base = [t if t not in (MATCH_QUERY, MATCH_KEY) else 8 for t in random_tokens(cfg["vocab"], length, 5)]
    places = [0, 1, 2, page - 1, page, page + 1, 2 * page - 1, 2 * page, 100, 255, 256, 257, length - 3, length - 2]
    config, weights = plain.read_folder(folder)
    for j in places:
        tokens = list(base)
        tokens[j], tokens[-1] = MATCH_KEY, MATCH_QUERY
        want = plain.forward(config, weights, tokens).numpy()
        without = list(tokens); without[j] = 9
        shift = np.abs(plain.forward(config, weights, without).numpy()[-1] - want[-1]).max()
        assert shift > 0.05 * np.abs(want[-1]).max(), "the crafted key does not stand out"
        cuts = {"prompt": [length], "alone": [length - 1, 1], "portions": [j + 1, length - j - 2, 1] if j < length - 2 else [length - 2, 2],
                "decoded": [max(j, 1)] + [1] * (length - max(j, 1))}
        for kind, cut in cuts.items():
            steps, p = [], 0
            for n in cut:
                if n <= 0:
                    continue
                steps.append({"step": len(steps), "entries": [{"id": "m", "tokens": tokens[p:p + n],
                                                              "want": [n - 1] if p + n == length else []}],
                              "end": ["m"] if p + n == length else []})
                p += n
            rows = replay_in_process(folder, dtype, steps, tmp_path / f"{dtype}{j}{kind}", block_size=page, max_tokens=384)
            compare(rows, {"m": want}, dtype, f"match at {j}, {kind}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype, folders):
    """One request slot and barely enough pages: each request gets the slot and pages its predecessor gave
    back, with the predecessor's state and keys still in them (the manager zeroes the state)."""
    name = "A"
    model = tw.load_model(folders[name], dtype, "cuda")
    cache = tw.CacheManager(model.cache_needs(), LINURAX_PAGE[name], 9, 1, 72, model.runtime.dtype, model.runtime.device,
                            prefix_cache=False)
    runner = ModelRunner(model, cache, 72, 1, cuda_graphs=False)
    config, weights = plain.read_folder(folders[name])
    for i, n in enumerate([70, 64, 3, 71]):
        tokens = random_tokens(config["vocab"], n, 40 + i)
        lease = cache.admit(None)
        assert lease.slot == 0
        cut = max(1, n // 2)
        cache.ensure(lease, cut)
        runner.step([StepEntry(lease.slot, tokens[:cut], 0, [])])
        cache.ensure(lease, n)
        got = runner.step([StepEntry(lease.slot, tokens[cut:], cut, list(range(n - cut)))]).cpu().numpy() if n > cut else None
        runner.check_status()
        cache.release(lease)
        cache.check_invariants()
        if got is not None:
            want = plain.forward(config, weights, tokens).numpy()
            compare({("r", cut + k): got[k] for k in range(n - cut)}, {"r": want}, dtype, f"request {i} in a used slot")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders, tmp_path):
    """Three hundred tokens one by one after a short prompt, through CUDA graphs where the runner has them."""
    name = "B"
    tokens = random_tokens(LINURAX_CONFIGS[name]["vocab"], 320, 77)
    want = plain.logits_of(folders[name], tokens).numpy()
    model = tw.load_model(folders[name], dtype, "cuda")
    cache = tw.CacheManager(model.cache_needs(), 16, 24, 2, 384, model.runtime.dtype, model.runtime.device, prefix_cache=False)
    runner = ModelRunner(model, cache, 64, 2, cuda_graphs=True)
    lease = cache.admit(None)
    cache.ensure(lease, 20)
    runner.step([StepEntry(lease.slot, tokens[:20], 0, [])])
    rows = {}
    for p in range(20, 320):
        cache.ensure(lease, p + 1)
        rows[("r", p)] = runner.step([StepEntry(lease.slot, [tokens[p]], p, [0])])[0].cpu().numpy().copy()
    runner.check_status()
    compare(rows, {"r": want}, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(name, dtype, folders):
    """``generate`` (scheduler, continuous batching, CUDA graphs, look-ahead) against the plain greedy loop;
    in bfloat16 every chosen token must be the plain implementation's best on that path, or nearly."""
    prompts = [random_tokens(LINURAX_CONFIGS[name]["vocab"], n, 60 + n) for n in (21, 5, 40)]
    model = tw.load_model(folders[name], dtype, "cuda")
    out = tw.generate(model, prompts, max_tokens=12, ignore_eos=True,
                      engine_config=tw.EngineConfig(block_size=LINURAX_PAGE[name], kv_blocks=40, max_context=128, max_active=2,
                                                    prefill_chunk=16))
    config, weights = plain.read_folder(folders[name])
    for p, o in zip(prompts, out):
        assert len(o) == 12
        logits = plain.forward(config, weights, p + o)
        for i, t in enumerate(o):
            row = logits[len(p) + i - 1]
            gap = float(row.max() - row[t])
            spread = float(row.std())
            assert gap <= (1e-4 if dtype == "float32" else 0.15) * spread, f"token {i} lies {gap:.3g} below the best (spread {spread:.3g})"
