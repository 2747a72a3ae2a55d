"""The Vugedra design in the engine against the plain implementation of `plain_vugedra.py`: every mechanism's
kernel alone (with inputs made so that a lost key, a wrong edge or a lost sink shows), then whole models in every
way of cutting a request into steps, mixed batches with pages and state slots used again, long decoding under
CUDA graphs, and greedy generation through the engine's own entry point and scheduler."""
import types

import numpy as np
import pytest
import torch

import plain_vugedra as pv
import replay_helpers as rh
import vugedra_models as vm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64

CASES = {"A": (vm.VUG_A, vm.VUG_A_PAGE, 3), "B": (vm.VUG_B, vm.VUG_B_PAGE, 5), "C": (vm.VUG_C, vm.VUG_C_PAGE, 9),
         "D": (vm.VUG_D, vm.VUG_D_PAGE, 11), "E": (vm.VUG_E, vm.VUG_E_PAGE, 13)}
# root mean square over the vocabulary of (difference minus its mean), as a fraction of the reference logits'
# spread; the float32 run is measured against the plain code in double precision
LIMIT = {"float32": 1e-4, "bfloat16": 0.12}


def model_of(case):
    cfg, page, seed = CASES[case]
    return cfg, page, vm.random_weights(cfg, seed)


def _spread_error(row, ref_row, spread):
    d = np.asarray(row, dtype=np.float64) - ref_row
    return float(np.sqrt(np.mean((d - d.mean()) ** 2))) / spread


class Reference:
    """Whole-sequence logits of the plain code in double precision, and for each position the error that rounding
    activations to bfloat16 alone causes there (the plain code run again with that rounding, and with the rounding
    jittered): a close call between two experts that a 16-bit run decides the other way is a jump that no
    implementation can avoid, and none can be held to more than a few times its own rounding."""

    def __init__(self, cfg, w, reqs, dtype):
        w64 = {k: v.double() for k, v in w.items()}
        self.rows = {r: pv.forward(cfg, w64, t).numpy() for r, t in reqs.items()}
        self.spread = float(np.sqrt(np.mean([np.var(v) for v in self.rows.values()])))
        self.dtype = dtype
        self.own = {}
        if dtype == "bfloat16":
            for r, t in reqs.items():
                runs = [pv.forward(cfg, w64, t, act=pv.bf16_round).numpy()]
                runs += [pv.forward(cfg, w64, t, act=pv.bf16_round_jittered(seed)).numpy() for seed in (1, 2)]
                self.own[r] = [max(_spread_error(x[p], self.rows[r][p], self.spread) for x in runs) for p in range(len(t))]

    def limit(self, r, pos):
        return max(LIMIT[self.dtype], 3.0 * self.own[r][pos]) if self.own else LIMIT[self.dtype]

    def error(self, row, r, pos):
        return _spread_error(row, self.rows[r][pos], self.spread)


def assert_close(got, ref, dtype, what):
    """float32: every position within the limit.  bfloat16: 3 positions in 100 may exceed theirs."""
    assert got, "nothing was compared"
    held, over = 0, []
    for (r, pos) in sorted(got):
        err, limit = ref.error(got[(r, pos)], r, pos), ref.limit(r, pos)
        if err > limit:
            over.append(f"{what}: request {r} position {pos}: {err:.3e} > {limit:.1e}")
        held += limit <= 2 * LIMIT[dtype]
    allowed = 0 if dtype == "float32" else max(1, int(0.03 * len(got)))
    assert len(over) <= allowed, "; ".join(over[:5])
    assert held >= 0.6 * len(got), "too few positions are well conditioned for this to be a test"


def requests(cfg, lengths, seed):
    return {f"r{i}": vm.random_tokens(cfg, n, seed * 100 + i) for i, n in enumerate(lengths)}


# ---- whole models, every cutting ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D", "E"])
def test_every_cutting_matches_plain(case, dtype):
    cfg, page, w = model_of(case)
    reqs = requests(cfg, [1, 2, 3, 37, 90, 150], seed=1)
    ref = Reference(cfg, w, reqs, dtype)
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=33)),
                        ("portions", rh.trace_portions(reqs, seed=2)),
                        ("mixed", rh.trace_mixed(reqs, seed=3, max_live=3))):
        # a pool just large enough, and three slots for six requests: pages and slots are used again
        runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=3)
        assert_close(rh.run_trace(runner, steps), ref, dtype, f"{case} {name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_window_and_kept_keys_over_pages(dtype):
    """600 tokens: the window of 130 keys passes over page borders in one step, in portions of many sizes and in 140
    decoded tokens, while the first 20 keys (a page and a quarter) stay; pages between them go back to the pool on
    the way, and the recurrent layers' scans run in chunks."""
    cfg, page, w = model_of("C")
    reqs = requests(cfg, [600, 300], seed=4)
    ref = Reference(cfg, w, reqs, dtype)
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=140)),
                        ("portions", rh.trace_portions(reqs, seed=5, sizes=(2, 61, 64, 65, 128, 257, 300)))):
        runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=2)
        assert_close(rh.run_trace(runner, steps), ref, dtype, name)


def test_long_prompt_with_attention_heads_of_128():
    """450 tokens in the 16-bit mode with attention heads of 128: portions that start in the middle of a page, a window
    of 140 keys with six kept ones, decoded tokens after them."""
    cfg, page, w = model_of("E")
    reqs = requests(cfg, [450, 260], seed=8)
    ref = Reference(cfg, w, reqs, "bfloat16")
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=40)),
                        ("portions", rh.trace_portions(reqs, seed=9, sizes=(2, 61, 127, 128, 129, 257)))):
        runner = rh.make_runner(cfg, w, "bfloat16", page, rh.peak_tokens(steps, round_to=page), max_requests=2)
        assert_close(rh.run_trace(runner, steps), ref, "bfloat16", name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_under_graphs(dtype):
    """Two prompt tokens, then 200 single-token steps of two requests side by side: steps of one shape are replayed as
    a captured graph, the recurrent states move on once per replay, the windows slide past the kept keys."""
    cfg, page, w = model_of("A")
    reqs = requests(cfg, [202, 180], seed=6)
    ref = Reference(cfg, w, reqs, dtype)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:2], "want": [0, 1]} for r, t in reqs.items()], "end": []}]
    for k in range(2, 202):
        live = [(r, t) for r, t in reqs.items() if k < len(t)]
        steps.append({"step": len(steps), "entries": [{"id": r, "tokens": [t[k]], "want": [0]} for r, t in live],
                      "end": [r for r, t in live if k == len(t) - 1]})
    runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=2)
    assert_close(rh.run_trace(runner, steps), ref, dtype, "long decoding")
    assert runner.graph_replays > 100


def test_batch_does_not_change_a_request():
    """The same request alone and beside others of other lengths: float32 logits agree to rounding."""
    cfg, page, w = model_of("B")
    reqs = requests(cfg, [64, 5, 33], seed=7)
    alone = {}
    for r, t in reqs.items():
        runner = rh.make_runner(cfg, w, "float32", page, 256, max_requests=3)
        alone.update(rh.run_trace(runner, rh.trace_whole({r: t})))
    runner = rh.make_runner(cfg, w, "float32", page, 256, max_requests=3)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()],
              "end": list(reqs)}]
    together = rh.run_trace(runner, steps)
    for key, row in alone.items():
        assert np.abs(row - together[key]).max() <= 2e-5 * max(1.0, np.abs(row).max()), key


def test_greedy_generation_through_the_engine_and_scheduler():
    """`PagedGenerateEngine.generate`: chunked prompts, decode batches, more requests than slots, a pool that forces
    preemption; the tokens are the plain code's greedy tokens."""
    from litellmengine_b200.engine import PagedGenerateEngine
    cfg, page, w = model_of("D")
    w64 = {k: v.double() for k, v in w.items()}
    prompts = [vm.random_tokens(cfg, n, 50 + i) for i, n in enumerate([9, 30, 3, 17, 22])]
    new = 12
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(new):
            ids.append(int(pv.forward(cfg, w64, ids)[-1].argmax()))
        want.append(ids[len(p):])
    runner = rh.make_runner(cfg, w, "float32", page, 64, max_requests=3, max_tokens_per_step=32)
    engine = PagedGenerateEngine(runner, chunk=8)
    got = engine.generate(prompts, new)
    assert got == want
    assert engine.scheduler.num_preemptions > 0
    runner.cache.check_invariants()


def test_trace_replay_and_prompt_command_on_a_model_folder(tmp_path):
    """`bin/trace_run` and `bin/run_prompt` on a folder written in the design's own format."""
    import json
    import os
    import subprocess
    import sys
    from litellmengine_b200.weights.safetensors_io import write_safetensors
    cfg, page, w = model_of("A")
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(folder / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    toks = vm.random_tokens(cfg, 40, 8)
    w64 = {k: v.double() for k, v in w.items()}
    ref = pv.forward(cfg, w64, toks).numpy()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:25], "want": [3, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[25:], "want": [14]}], "end": ["a"]}]
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32",
                          "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    spread = float(np.std(ref))
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    for row, pos in ((got0[0], 3), (got0[1], 24), (got1[0], 39)):
        assert _spread_error(row, ref[pos], spread) < 1e-4
    prompt = toks[:17]
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(pv.forward(cfg, w64, ids)[-1].argmax()))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "run_prompt"), "--model", str(folder), "--input-ids",
                           ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert proc.stdout.strip().split("\n")[-1] == ",".join(map(str, ids[len(prompt):]))


# ---- mechanisms alone -------------------------------------------------------------------------------
def _ops():
    from litellmengine_b200.csrc import ops
    return ops


def _i32(x):
    return torch.as_tensor(x, dtype=torch.int32, device=DEV)


def _f32(t):
    return t.float().to(DEV).contiguous()


def _batch(portions):
    """What the kernels read of a step: `portions` = [(slot, first position, tokens)] in batch order."""
    pos, ent, slots, starts, lens = [], [], [], [], []
    for e, (slot, p0, n) in enumerate(portions):
        starts.append(len(pos))
        lens.append(n)
        slots.append(slot)
        pos += list(range(p0, p0 + n))
        ent += [e] * n
    return types.SimpleNamespace(positions=_i32(pos), token_entry=_i32(ent), entry_slot=_i32(slots), entry_q_start=_i32(starts),
                                 entry_q_len=_i32(lens), num_tokens=len(pos))


@pytest.mark.parametrize("H", [40, 36, 30, 1024])
def test_tanh_norm_around_the_residual_add(H):
    """v = h + post(y), h <- v, out = pre(v): every way the arrangement uses the kernel, for row lengths that take
    sixteen-byte accesses and that do not; y as one matrix, as 16-bit, as the k-splits of a product; picked rows."""
    ops = _ops()
    T = 11
    g = torch.Generator().manual_seed(H)
    h0, y = torch.randn(T, H, generator=g, dtype=F64), torch.randn(3, T, H, generator=g, dtype=F64) * 2

    def norm(seed):
        gg = torch.Generator().manual_seed(seed)
        return {"n": 1 + 0.2 * torch.randn(H, generator=gg, dtype=F64), "n.alpha": torch.tensor(0.4 + seed / 10.0, dtype=F64),
                "n.b": 0.3 * torch.randn(H, generator=gg, dtype=F64)}
    post, pre = norm(3), norm(7)
    dev = lambda n: (_f32(n["n.alpha"].reshape(1)), _f32(n["n"]), _f32(n["n.b"]))
    # nothing pending: the first layer's input norm
    h = _f32(h0)
    out = ops.tanh_norm(h, None, None, dev(pre), torch.float32)
    assert (out.double().cpu() - pv.tanh_norm(h0, pre, "n")).abs().max() < 2e-6 and torch.equal(h.cpu(), h0.float())
    # a sublayer's output through its norm, the add, the next norm; y as float32, as k-splits, as 16-bit
    want_h = h0 + pv.tanh_norm(y.sum(0), post, "n")
    for form in ("one", "splits", "bf16"):
        h = _f32(h0)
        if form == "one":
            given = _f32(y.sum(0))
        elif form == "splits":
            given = ops.PartialSum(_f32(y))
        else:
            given = y.sum(0).to(torch.bfloat16).to(DEV)
            want_h = h0 + pv.tanh_norm(given.double().cpu(), post, "n")
        out = ops.tanh_norm(h, given, dev(post), dev(pre), torch.bfloat16 if form == "bf16" else torch.float32)
        assert (h.double().cpu() - want_h).abs().max() < 5e-6, form
        assert (out.double().cpu() - pv.tanh_norm(want_h, pre, "n")).abs().max() < (2e-2 if form == "bf16" else 5e-6), form
    # the add alone (nothing behind it), and picked rows for a model's last norm (the stream is left alone)
    h = _f32(h0)
    assert ops.tanh_norm(h, _f32(y[0]), dev(post), None) is None
    assert (h.double().cpu() - (h0 + pv.tanh_norm(y[0], post, "n"))).abs().max() < 5e-6
    h, rows = _f32(h0), [7, 0, 7, 10]
    out = ops.tanh_norm(h, _f32(y[1]), dev(post), dev(pre), torch.float32, rows=_i32(rows))
    want = pv.tanh_norm(h0 + pv.tanh_norm(y[1], post, "n"), pre, "n")[rows]
    assert (out.double().cpu() - want).abs().max() < 5e-6 and torch.equal(h.cpu(), h0.float())


def _paged(T, page, nkv, dk, dv, dtype, shuffle_seed=0):
    """One request of T tokens in slot 1 of 3, its pages scattered over a pool."""
    n = -(-T // page)
    pool = n + 5
    order = np.random.RandomState(shuffle_seed).permutation(pool)[:n]
    table = torch.full((3, n + 2), -1, dtype=torch.int32)
    table[1, :n] = torch.as_tensor(order, dtype=torch.int32)
    keys = torch.zeros(pool, nkv, page, dk, dtype=dtype, device=DEV)
    values = torch.zeros(pool, nkv, page, dv, dtype=dtype, device=DEV) if dv else None
    return keys, values, table.to(DEV), order


@pytest.mark.parametrize("window,keep,dims,scaling", [(None, 0, 8, None), (1, 0, 12, (4.0, 16, 4.0, 0.5)), (7, 3, 4, None),
                                                      (64, 17, 12, (2.0, 64, 8.0, 1.0)), (65, 16, 0, None), (5, 40, 6, (8.0, 8, 2.0, 0.25))])
def test_attention_projection_norm_rotation_window_kept_keys_and_sink(window, keep, dims, scaling):
    """The kernels between the projections of an attention layer, on projections given as numbers: biases, the norm over
    the whole projection, the rotation of neighbouring pairs with stretched frequencies, the page write; then attention
    with a window, kept first keys and the sink.  One key is turned towards a late query so that it would win by far, and
    placed just inside and just outside that query's window, just inside and just outside the kept keys, at a page's last
    and first place and at the sequence's first token.  The last query's own scores are made very negative, so that
    the sink takes nearly all of its weight.  Prompt rows and single tokens against the plain functions."""
    ops = _ops()
    T, page, H, G, D, V, scale, eps = 150, 16, 6, 2, 12, 20, 0.3, 1e-5
    g = torch.Generator().manual_seed(5)
    proj = torch.randn(T, H * D + G * D + G * V + H, generator=g, dtype=F64)
    w = {"q.b": 0.2 * torch.randn(H * D, generator=g, dtype=F64), "k.b": 0.2 * torch.randn(G * D, generator=g, dtype=F64),
         "v.b": 0.2 * torch.randn(G * V, generator=g, dtype=F64), "q.norm": 1 + 0.1 * torch.randn(H * D, generator=g, dtype=F64),
         "k.norm": 1 + 0.1 * torch.randn(G * D, generator=g, dtype=F64)}
    rot = None
    if dims:
        rot = {"base": 300.0, "dims": dims}
        if scaling:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mask = {"size": window, "keep_first": keep} if window else None
    ko, vo, go = H * D, H * D + G * D, H * D + G * D + G * V

    def qkv(p):
        q = pv.rms_unit(p[:, :ko] + w["q.b"], eps) * w["q.norm"]
        k = pv.rms_unit(p[:, ko:vo] + w["k.b"], eps) * w["k.norm"]
        v = p[:, vo:go] + w["v.b"]
        pos = list(range(T))
        return (pv.rotate_pairs(q.view(T, H, D), pos, rot), pv.rotate_pairs(k.view(T, G, D), pos, rot), v.view(T, G, V))

    def plain(p, sink=True):
        q, k, v = qkv(p)
        s = (q.permute(1, 0, 2) @ k.permute(1, 0, 2).repeat_interleave(H // G, 0).transpose(1, 2)) * scale
        o = pv.softmax_core(s, v.permute(1, 0, 2).repeat_interleave(H // G, 0), pv.visible_keys(T, mask), sink=sink)
        return (o.permute(1, 0, 2) * torch.sigmoid(p[:, go:])[:, :, None]).reshape(T, H * V)

    # a key that points where head 0 of a late query looks (before norm and rotation that is only roughly so; 6 times over)
    probes = [(149, (window or 150) - 1), (148, window or 148), (130, (window or 131) - 1), (141, 141 - 16), (140, 140 - 15), (120, 120),
              (147, 147 - max(keep - 1, 0)), (146, 146 - keep)]
    for i, back in probes:
        j = i - back
        if 0 <= j < i:
            proj[j, ko:ko + D] = proj[i, :D] * 6.0
    proj[T - 1, :ko] *= -1.0                    # the last query looks away from everything it sees, itself included:
    proj[T - 1, ko:vo] = proj[T - 1, :D].repeat(G) * -5.0           # the sink takes the weight
    ref = plain(proj)
    assert (ref - plain(proj, sink=False)).abs().max() > 0.05          # the sink matters
    from litellmengine_b200.config.specs import PositionSpec
    from litellmengine_b200.parts.registry import lookup
    import litellmengine_b200.parts.position  # noqa: F401  (registers the kinds)
    rotation = None
    if dims:
        params = (("scaling", scaling), ("magnitude", 0.1 * np.log(scaling[0]) + 1.0)) if scaling else ()
        rotation = lookup("position", "rope_pairs")(PositionSpec("rope_pairs", 300.0, dims, params), D, DEV).kernel_args()
    for dtype, tol in ((torch.float32, 3e-5), (torch.bfloat16, 0.06)):
        for portions in ([(1, 0, T)], [(1, 0, 70), (1, 70, 2), (1, 72, 77)] + [(1, p, 1) for p in range(149, 150)]):
            keys, values, block_table, order = _paged(T, page, G, D, V, dtype, 2)
            out = torch.zeros(T, H * V, dtype=dtype, device=DEV)
            status = torch.zeros(2, dtype=torch.int32, device=DEV)
            at = 0
            for slot, p0, n in portions:                        # step by step, as a request would run
                b = _batch([(slot, p0, n)])
                rows = _f32(proj[p0:p0 + n])
                q = ops.attention_prepare(rows, 0, ko, vo, (_f32(w["q.b"]), _f32(w["k.b"]), _f32(w["v.b"])), _f32(w["q.norm"]),
                                          _f32(w["k.norm"]), "projection", eps, None, keys, values, b.positions, b.token_entry,
                                          b.entry_slot, block_table, H, G, D, V, page, status, dtype, rotation=rotation)
                o = torch.zeros(n, H * V, dtype=dtype, device=DEV)
                ops.paged_attention_generic_kv(q, keys, values, b.positions, b.token_entry, b.entry_slot, block_table, H, G, D, V,
                                               page, window, scale, status, o, gate=rows, gate_off=go, gate_per_head=True,
                                               keep_first=keep, sink=0.0)
                out[p0:p0 + n] = o
                at += n
            assert at == T and status.tolist() == [0, 0]
            assert (out.double().cpu() - ref).abs().max() < tol, (window, keep, dims, dtype, len(portions))
    if window:                      # the edges matter: one key further out, or one more kept, and the result is another
        mask = {"size": window + 1, "keep_first": keep}
        assert (ref - plain(proj)).abs().max() > 0.02
        mask = {"size": window, "keep_first": keep + 1}
        assert (ref - plain(proj)).abs().max() > 0.02


@pytest.mark.parametrize("dims,scaling", [(8, None), (4, (4.0, 16, 4.0, 0.5)), (0, None)])
def test_latent_attention_with_pair_rotation_and_a_gate_per_head(dims, scaling):
    """The latent attention mixer's kernels with the rotation of neighbouring pairs (stretched or not, over a part of the
    rotated entries or all of them) against per-head keys and values made plainly; one cached row is turned towards a
    late query and placed far back, at a page's border and at the sequence's start."""
    ops = _ops()
    T, page, H, D, P, V, Q, R, scale, eps, base = 150, 16, 3, 12, 8, 20, 28, 24, 0.3, 1e-5, 300.0
    g = torch.Generator().manual_seed(5)
    u = torch.randn(T, 16, generator=g, dtype=F64)
    m = {"heads": H, "dim": D, "rot_dim": P, "vdim": V, "kv_rank": R, "q_rank": Q, "scale": scale}
    if dims:
        m["rot"] = {"base": base, "dims": dims}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    w = {"dq": torch.randn(Q, 16, generator=g, dtype=F64) / 4, "dq.norm": 1 + 0.1 * torch.randn(Q, generator=g, dtype=F64),
         "uq": torch.randn(H * (D + P), Q, generator=g, dtype=F64) * Q ** -0.5 * 2, "dkv": torch.randn(R + P, 16, generator=g, dtype=F64) / 4,
         "dkv.norm": 1 + 0.1 * torch.randn(R, generator=g, dtype=F64), "uk": torch.randn(H * D, R, generator=g, dtype=F64) * R ** -0.5,
         "uv": torch.randn(H * V, R, generator=g, dtype=F64) * R ** -0.5, "g": torch.randn(H, 16, generator=g, dtype=F64),
         "o": torch.eye(H * V, dtype=F64)}
    ref = pv.latent_attention(u, w, "", m, eps)
    from litellmengine_b200.config.specs import PositionSpec
    from litellmengine_b200.parts.registry import lookup
    import litellmengine_b200.parts.position  # noqa: F401
    inv_freq, rd, mag, pairs = None, 0, 1.0, False
    if dims:
        params = (("scaling", scaling), ("magnitude", 0.1 * np.log(scaling[0]) + 1.0)) if scaling else ()
        inv_freq, rd, mag, pairs = lookup("position", "rope_pairs")(PositionSpec("rope_pairs", base, dims, params), P, DEV).kernel_args()
    dq, dkv, gate = u @ w["dq"].T, u @ w["dkv"].T, u @ w["g"].T
    for dtype, tol in ((torch.float32, 3e-5), (torch.bfloat16, 0.06)):
        keys, _, block_table, order = _paged(T, page, 1, R + P, 0, dtype, 2)
        proj = torch.zeros(T, 5 + Q + R + P + H, dtype=torch.float32, device=DEV)
        proj[:, 5:5 + Q], proj[:, 5 + Q:5 + Q + R + P], proj[:, 5 + Q + R + P:] = _f32(dq), _f32(dkv), _f32(gate)
        b = _batch([(1, 0, T)])
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        cq = ops.latent_prepare(proj, 5, 5 + Q, Q, R, P, rd, _f32(w["dq.norm"]), _f32(w["dkv.norm"]), eps, inv_freq, keys, b, block_table,
                                page, status, dtype, rot_pairs=pairs, rot_mag=mag)
        q32 = (cq.double().cpu() @ w["uq"].T).float().to(DEV)
        qn_dev, packed = ops.latent_q_split(q32, b.positions, inv_freq, H, D, P, R, rd, dtype, rot_pairs=pairs, rot_mag=mag)
        folded = torch.bmm(qn_dev.double(), w["uk"].view(H, D, R).to(DEV))
        packed.view(T, H, R + P)[:, :, :R] = folded.permute(1, 0, 2).to(dtype)
        lat = torch.zeros(T, H * R, dtype=dtype, device=DEV)
        ops.paged_attention_generic_kv(packed, keys, None, b.positions, b.token_entry, b.entry_slot, block_table, H, 1, R + P, R,
                                       page, None, scale, status, lat, values_in_keys=True)
        assert status.tolist() == [0, 0]
        heads = torch.einsum("thr,hvr->thv", lat.double().cpu().view(T, H, R), w["uv"].view(H, V, R)).reshape(T, H * V).to(dtype).to(DEV)
        ops.gate_mul(heads, proj, 5 + Q + R + P, heads, 0, "sigmoid", per_head=V)
        assert (heads.double().cpu() - ref).abs().max() < tol, (dims, dtype)


@pytest.mark.parametrize("E,I,top,W", [(5, 1, 2, 40), (3, 2, 5, 30), (8, 0, 3, 64), (6, 3, 1, 36), (40, 4, 6, 48)])
def test_router_softmax_correction_and_outputs_without_an_expert(E, I, top, W):
    """The router against the plain rule: softmax over all outputs, the choice by score + correction, the weights from the
    scores alone; the correction is large enough to change choices.  The dense row, the lists and a token's own share."""
    ops = _ops()
    T = 53
    g = torch.Generator().manual_seed(E * 10 + I)
    x = torch.randn(T, W, generator=g, dtype=F64)
    w = {"router": torch.randn(E + I, W, generator=g, dtype=F64) * W ** -0.5 * 2, "correction": 0.3 * torch.randn(E + I, generator=g, dtype=F64)}
    pick, weight = pv.route(x, w, "", {"top": top})
    plain_pick, _ = pv.route(x, dict(w, correction=w["correction"] * 0), "", {"top": top})
    assert (pick.sort(1).values != plain_pick.sort(1).values).any() or top == E + I      # the correction matters
    got = ops.moe_route(_f32(x), _f32(w["router"]), top, None, 1.0, lists=True, score="softmax", correction=_f32(w["correction"]),
                        identity=I)
    dense, ids, wts = got[:3]
    want_dense, want_own = torch.zeros(T, E, dtype=F64), torch.zeros(T, dtype=F64)
    for t in range(T):
        for e, a in zip(pick[t].tolist(), weight[t].tolist()):
            if e < E:
                want_dense[t, e] = a
            else:
                want_own[t] += a
    assert (dense.double().cpu() - want_dense).abs().max() < 1e-6
    if I:
        assert (got[3].double().cpu() - want_own).abs().max() < 1e-6
    for t in range(T):
        mine = {int(e): float(a) for e, a in zip(ids[t].tolist(), wts[t].tolist()) if e >= 0}
        assert set(mine) == {e for e in pick[t].tolist() if e < E}
        assert all(abs(mine[e] - float(want_dense[t, e])) < 1e-6 for e in mine)


@pytest.mark.parametrize("dtype,T", [("float32", 3), ("float32", 50), ("bfloat16", 2), ("bfloat16", 20), ("bfloat16", 70)])
def test_routed_feed_forward_every_way_it_runs(dtype, T):
    """The routed feed-forward part (few tokens: only the chosen experts are read; prompt portions in 16 bits: tokens
    sorted by expert; else all experts in one product) with outputs that are no experts and a shared expert of another
    size, against the plain function."""
    from litellmengine_b200.config.specs import FeedForwardSpec
    from litellmengine_b200.parts.feed_forward import RoutedExperts
    W, E, I, top, ff, shared = 48, 12, 2, 3, 16, 24
    g = torch.Generator().manual_seed(T)
    bf = lambda t: t.to(torch.bfloat16).double()
    x = bf(torch.randn(T, W, generator=g, dtype=F64))
    w = {"router": bf(torch.randn(E + I, W, generator=g, dtype=F64) * W ** -0.5 * 3), "correction": bf(0.2 * torch.randn(E + I, generator=g, dtype=F64))}
    for name, n in [(f"e{e}.", ff) for e in range(E)] + [("shared.", shared)]:
        w[name + "gate"], w[name + "up"] = (bf(torch.randn(n, W, generator=g, dtype=F64) * W ** -0.5) for _ in range(2))
        w[name + "down"] = bf(torch.randn(W, n, generator=g, dtype=F64) * n ** -0.5)
    mlp = {"router": {"experts": E, "identity": I, "top": top}, "shared": {"ff": shared}}
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    ref = pv.routed_ff(x, w, "", mlp, act=pv.bf16_round if dtype == "bfloat16" else pv.identity)
    part = RoutedExperts(FeedForwardSpec(kind="moe", intermediate_size=ff, params=(
        ("experts", E), ("top", top), ("groups", None), ("score", "softmax"), ("correction", True), ("identity", I),
        ("activation", "silu"), ("shared", shared))), W, tdt, DEV)
    part.load({k: (v.to(tdt) if v.dim() == 2 and k != "router" else v.float()).to(DEV) for k, v in w.items()})
    got = _ops().as_tensor(part.forward(x.to(tdt).to(DEV)))
    assert (got.double().cpu() - ref).abs().max() < (3e-5 if dtype == "float32" else 0.05) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("d,group,window,keep", [(64, 2, 100, 5), (128, 1, 64, 70), (128, 2, 140, 6), (128, 4, 257, 129), (128, 8, None, 0),
                                                 (64, 4, 30, 0)])
def test_tensor_core_attention_with_kept_keys_and_sink(d, group, window, keep):
    """The kernels that a 16-bit run takes at head sizes 64 and 128: a prompt portion that starts in the middle of a page
    with keys before it (row tiles of 128 whose window begins several key tiles after the kept keys), and single tokens in
    the split-key decode kernel, where one more split walks the kept keys.  Keys that would win by far sit among the kept
    ones, just behind them, and at the window's first and just before it."""
    ops = _ops()
    N, past, page, G, scale = 420, 37, 16, 2, 0.2
    H, T = G * group, N - past
    g = torch.Generator().manual_seed(d + group)
    q, k, v = (torch.randn(N, n, d, generator=g, dtype=F64) for n in (H, G, G))
    w = window or N
    for i, j in ((419, max(keep - 1, 0)), (418, keep), (417, 417 - w + 1), (416, 416 - w), (300, 3), (299, max(299 - w, 0))):
        k[j] = q[i, ::group] * (40.0 / d)          # a score of about ten
    q[N - 2] = -q[N - 2].abs() * 3                  # a query that looks away from all it sees: the sink takes its weight
    k[max(N - 2 - w + 1, 0):N - 1] = k[max(N - 2 - w + 1, 0):N - 1].abs()
    k[:keep] = k[:keep].abs()
    q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    mask = {"size": window, "keep_first": keep} if window else None
    vis = pv.visible_keys(N, mask)[past:]
    kh, vh = (t.permute(1, 0, 2).repeat_interleave(group, 0) for t in (k, v))
    scores = (q[past:].permute(1, 0, 2) @ kh.transpose(1, 2)) * scale
    ref = pv.softmax_core(scores, vh, vis, sink=True).permute(1, 0, 2)
    assert ref[N - 2 - past].abs().max() < 0.2 * ref.abs().max()        # the sink took nearly all of that query's weight
    order = np.random.RandomState(2).permutation(N // page + 6)[:-(-N // page)]
    block_table = torch.full((3, len(order) + 2), -1, dtype=torch.int32)
    block_table[1, :len(order)] = torch.as_tensor(order, dtype=torch.int32)
    block_table = block_table.to(DEV)
    cache = torch.zeros(N // page + 6, 2, G, page, d, dtype=torch.bfloat16, device=DEV)
    for j in range(N):
        cache[order[j // page], 0, :, j % page] = k[j].to(torch.bfloat16).to(DEV)
        cache[order[j // page], 1, :, j % page] = v[j].to(torch.bfloat16).to(DEV)
    qd = q[past:].reshape(T, -1).to(torch.bfloat16).to(DEV)
    out = torch.zeros(T, H * d, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    tiles = _i32([(0, r0) for r0 in range(0, T, ops.PREFILL_TILE_ROWS)])
    ops.paged_attention_prefill_biased(qd, out, 0, cache, tiles, tiles.shape[0], _i32([1]), _i32([0]), _i32([T]), _i32([N]),
                                       block_table, H, G, d, page, window, scale, status, keep_first=keep, sink=0.0)
    assert status.tolist() == [0, 0]
    assert (out.double().cpu().view(T, H, d) - ref).abs().max() < 0.06
    assert ops.fast_attention_supported(d, group)
    for splits in (1, 3):
        a = torch.zeros(T, H * d, dtype=torch.bfloat16, device=DEV)
        picked = [T - 1, T - 2, T - 3, T - 4, 5, 263, 262]
        ops.paged_attention_decode(qd, a, cache, _i32(picked + [-1]), len(picked) + 1, _i32(list(range(past, N))), _i32([0] * T),
                                   _i32([1]), block_table, H, G, d, page, window, scale, splits, status, keep_first=keep, sink=0.0)
        assert status.tolist() == [0, 0]
        assert (a.double().cpu().view(T, H, d)[picked] - ref[picked]).abs().max() < 0.06, splits
    # the edges matter: without the kept keys, or with ordinary softmax, the result is another
    if window and keep:
        other = pv.softmax_core(scores, vh, pv.visible_keys(N, {"size": window})[past:], sink=True).permute(1, 0, 2)
        assert (other - ref).abs().max() > 0.05
    assert (pv.softmax_core(scores, vh, vis, sink=False).permute(1, 0, 2) - ref).abs().max() > 0.1


@pytest.mark.parametrize("H,D,V,tau", [(2, 8, 16, 1.0), (3, 16, 8, 4.0), (1, 48, 64, 16.0), (2, 128, 128, 8.0), (5, 4, 6, 32.0)])
def test_gated_linear_attention_in_one_pass_in_portions_and_token_by_token(H, D, V, tau):
    """The recurrent mixer's kernels on projections made from given weights, against the plain token-by-token function:
    the decays from the low-rank projection (a channel whose bias keeps it from ever decaying carries an impulse from the
    first token to the last; one whose bias makes it forget at once loses it), the recurrence in one pass, in portions
    that carry the state in the request's slot (down to two tokens and one), and through the kernel of decode steps,
    which makes the decays itself; the state left behind is checked too."""
    ops = _ops()
    T, Wd, rank, eps = 203, 24, 5, 1e-5
    g = torch.Generator().manual_seed(H * 100 + D)
    u = torch.randn(T, Wd, generator=g, dtype=F64)
    w = {"q": torch.randn(H * D, Wd, generator=g, dtype=F64) * Wd ** -0.5, "k": torch.randn(H * D, Wd, generator=g, dtype=F64) * Wd ** -0.5,
         "v": torch.randn(H * V, Wd, generator=g, dtype=F64) * Wd ** -0.5, "g": torch.randn(H * V, Wd, generator=g, dtype=F64) * Wd ** -0.5,
         "a1": torch.randn(rank, Wd, generator=g, dtype=F64) * Wd ** -0.5, "a2": torch.randn(H * D, rank, generator=g, dtype=F64),
         "a2.b": torch.randn(H * D, generator=g, dtype=F64) * 2, "norm": 1 + 0.1 * torch.randn(V, generator=g, dtype=F64),
         "o": torch.eye(H * V, dtype=F64)}
    w["a2"][0], w["a2.b"][0] = 0.0, 60.0          # never decays
    w["a2"][1], w["a2.b"][1] = 0.0, -60.0 * tau   # forgets at once
    u[0] *= 4.0                                   # an impulse at the first token
    m = {"heads": H, "dim": D, "vdim": V, "tau": tau}
    ref, s_ref = pv.gla(u, w, "", m, eps)
    cols = [u @ w[n].T for n in ("q", "k", "v", "g", "a1")]
    proj = torch.cat(cols, dim=1).float()
    offs = (0, H * D, 2 * H * D, 2 * H * D + H * V)
    a_off = 2 * H * D + 2 * H * V
    w2t, b2, nw = _f32(w["a2"].t()), _f32(w["a2.b"]), _f32(w["norm"])
    slots = _i32([2])

    def run(cuts, step=False):
        state = torch.zeros((4, H, D, V), dtype=torch.float32, device=DEV)
        state[1] = 7.0                                            # another request's state stays untouched
        out = torch.zeros((T, H * V), dtype=torch.float32, device=DEV)
        pd = proj.to(DEV)
        at = 0
        for n in cuts:
            rows = pd[at:at + n].contiguous()
            if step and n == 1:
                ops.gla_step(rows, offs, None, nw, eps, D ** -0.5, 1.0, out[at:at + n], 0, state, slots, _i32([0]), 1, H, D, V,
                             decay=(a_off, rank, w2t, b2, tau))
            else:
                alpha = ops.gla_decay(rows, a_off, rank, w2t, b2, tau)
                ops.gla_scan(rows, offs, alpha, nw, eps, D ** -0.5, 1.0, out[at:at + n], 0, state, slots, _i32([0]), _i32([n]), None, 1,
                             ops.GLA_FULL, None, None, H, D, V)
            at += n
        assert at == T and float((state[1] - 7.0).abs().max()) == 0 and float(state[0].abs().max()) == 0
        return out.double().cpu(), state[2].double().cpu()

    scale = max(1.0, float(ref.abs().max()))
    for what, (got, s) in (("one pass", run([T])), ("portions", run([2, 1, 16, 17, 2, 64, 70, 31])),
                           ("a portion, then the decode kernel token by token", run([33] + [1] * (T - 33), step=True))):
        assert (got - ref).abs().max() < 3e-5 * scale, what
        assert (s - s_ref).abs().max() < 3e-5 * max(1.0, float(s_ref.abs().max())), what
    flat = s_ref.reshape(H * D, V)
    assert flat[0].abs().max() > 10 * flat[1].abs().max()        # the impulse is kept by one channel and forgotten by the other
