"""The Komazen design in the engine against the plain implementation of `plain_komazen.py`: every mechanism's
kernel alone (with inputs made so that a lost key, a wrong edge or a lost row shows), then whole models in every
way of cutting a request into steps, mixed batches with pages and state slots used again, long decoding under
CUDA graphs, and greedy generation through the engine's own entry point and scheduler."""
import types

import numpy as np
import pytest
import torch

import komazen_models as km
import plain_komazen as pk
import replay_helpers as rh

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64

CASES = {"A": (km.KOMA_A, km.KOMA_A_PAGE, 3), "B": (km.KOMA_B, km.KOMA_B_PAGE, 5), "C": (km.KOMA_C, km.KOMA_C_PAGE, 9),
         "D": (km.KOMA_D, km.KOMA_D_PAGE, 11), "E": (km.KOMA_E, km.KOMA_E_PAGE, 13), "F": (km.KOMA_F, km.KOMA_F_PAGE, 17)}
# root mean square over the vocabulary of (difference minus its mean), as a fraction of the reference logits'
# spread; the float32 run is measured against the plain code in double precision
LIMIT = {"float32": 1e-4, "bfloat16": 0.12}


def model_of(case):
    cfg, page, seed = CASES[case]
    return cfg, page, km.random_weights(cfg, seed)


def _spread_error(row, ref_row, spread):
    d = np.asarray(row, dtype=np.float64) - ref_row
    return float(np.sqrt(np.mean((d - d.mean()) ** 2))) / spread


class Reference:
    """Whole-sequence logits of the plain code in double precision, and for each position the error that rounding
    activations to bfloat16 alone causes there (the plain code run again with that rounding, and with the rounding
    jittered): a norm after every sum amplifies what a peaked softmax does with a rounded score, and no
    implementation in bfloat16 can be held to more than a few times that."""

    def __init__(self, cfg, w, reqs, dtype):
        w64 = {k: v.double() for k, v in w.items()}
        self.rows = {r: pk.forward(cfg, w64, t).numpy() for r, t in reqs.items()}
        self.spread = float(np.sqrt(np.mean([np.var(v) for v in self.rows.values()])))
        self.dtype = dtype
        self.own = {}
        if dtype == "bfloat16":
            for r, t in reqs.items():
                runs = [pk.forward(cfg, w64, t, act=pk.bf16_round).numpy()]
                runs += [pk.forward(cfg, w64, t, act=pk.bf16_round_jittered(seed)).numpy() for seed in (1, 2)]
                self.own[r] = [max(_spread_error(x[p], self.rows[r][p], self.spread) for x in runs) for p in range(len(t))]

    def limit(self, r, pos):
        return max(LIMIT[self.dtype], 3.0 * self.own[r][pos]) if self.own else LIMIT[self.dtype]

    def error(self, row, r, pos):
        return _spread_error(row, self.rows[r][pos], self.spread)


def assert_close(got, ref, dtype, what):
    """float32: every position within the limit.  bfloat16: 2 positions in 100 may exceed theirs."""
    assert got, "nothing was compared"
    held, over = 0, []
    for (r, pos) in sorted(got):
        err, limit = ref.error(got[(r, pos)], r, pos), ref.limit(r, pos)
        if err > limit:
            over.append(f"{what}: request {r} position {pos}: {err:.3e} > {limit:.1e}")
        held += limit <= 2 * LIMIT[dtype]
    allowed = 0 if dtype == "float32" else max(1, int(0.02 * len(got)))
    assert len(over) <= allowed, "; ".join(over[:5])
    assert held >= 0.7 * len(got), "too few positions are well conditioned for this to be a test"


def requests(cfg, lengths, seed):
    return {f"r{i}": km.random_tokens(cfg, n, seed * 100 + i) for i, n in enumerate(lengths)}


# ---- whole models, every cutting ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D", "E", "F"])
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
def test_long_prompt_and_window_over_pages(dtype):
    """600 tokens: the window of 130 keys (and its reader's of 33) passes over page borders in one step, in portions
    of many sizes and in 140 decoded tokens; pages behind the widest window go back to the pool on the way."""
    cfg, page, w = model_of("C")
    reqs = requests(cfg, [600, 300], seed=4)
    ref = Reference(cfg, w, reqs, dtype)
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=140)),
                        ("portions", rh.trace_portions(reqs, seed=5, sizes=(2, 61, 64, 65, 128, 257, 300)))):
        runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=2)
        assert_close(rh.run_trace(runner, steps), ref, dtype, name)


def test_long_prompt_through_the_tensor_core_attention_kernels():
    """450 tokens with attention heads of 128 in bfloat16: row tiles of 128 that walk up to four tiles of 128 keys with the
    bias table renewed for each, portions that start in the middle of a page and of a tile, decoded tokens after them."""
    cfg, page, w = model_of("F")
    reqs = requests(cfg, [450, 260], seed=8)
    ref = Reference(cfg, w, reqs, "bfloat16")
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=40)),
                        ("portions", rh.trace_portions(reqs, seed=9, sizes=(2, 61, 127, 128, 129, 257)))):
        runner = rh.make_runner(cfg, w, "bfloat16", page, rh.peak_tokens(steps, round_to=page), max_requests=2)
        assert_close(rh.run_trace(runner, steps), ref, "bfloat16", name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_under_graphs(dtype):
    """Two prompt tokens, then 200 single-token steps of two requests side by side: steps of one shape are replayed as
    a captured graph, the kept rows of the convolutions move on once per replay, the windows slide."""
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
    prompts = [km.random_tokens(cfg, n, 50 + i) for i, n in enumerate([9, 30, 3, 17, 22])]
    new = 12
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(new):
            ids.append(int(pk.forward(cfg, w64, ids)[-1].argmax()))
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
    toks = km.random_tokens(cfg, 40, 8)
    w64 = {k: v.double() for k, v in w.items()}
    ref = pk.forward(cfg, w64, toks).numpy()
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
        ids.append(int(pk.forward(cfg, w64, ids)[-1].argmax()))
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


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_input_convolution_and_norm_after_the_sum_in_every_cutting(taps):
    """Two sequences run through convolution, then norm(alpha x + y) (which keeps the rows the next step's convolution
    wants): whole, in portions down to one token, interleaved in one batch, with a slot that held another sequence
    before.  Against the plain formulas."""
    ops = _ops()
    W, eps, alpha = 44, 1e-5, 1.7
    g = torch.Generator().manual_seed(taps)
    lens = {0: 23, 2: 17}
    x = {s: torch.randn(n, W, generator=g, dtype=F64) * 2 for s, n in lens.items()}
    y = {s: torch.randn(n, W, generator=g, dtype=F64) for s, n in lens.items()}
    w = torch.randn(W, taps, generator=g, dtype=F64) * 0.5
    wn = 1 + 0.1 * torch.randn(W, generator=g, dtype=F64)
    ref_u = {s: pk.input_convolution(x[s], w) for s in lens}
    ref_x = {s: pk.rms_norm(alpha * x[s] + y[s], wn, eps) for s in lens}
    f32 = lambda t: t.float().to(DEV).contiguous()
    schedules = ([[(0, 23), (2, 17)]],
                 [[(0, 1), (2, 2)], [(0, 1)], [(0, 2), (2, 1)], [(2, 14), (0, 19)]],
                 [[(2, 5), (0, 3)], [(2, 12)], [(0, 20)]])
    for steps in schedules:
        kept = torch.full((4, 2, taps - 1, W), 99.0, device=DEV)       # [slots, sublayers, rows, W]; sublayer 1 is used
        kept[[0, 2]] = 0                                                # an admitted request starts from zero rows
        ring = kept[:, 1] if taps > 1 else None
        at = {s: 0 for s in lens}
        for step in steps:
            placed = [(sl, at[sl], n) for sl, n in step]
            b = _batch(placed)
            h = f32(torch.cat([x[sl][p0:p0 + n] for sl, p0, n in placed]))
            u = ops.short_conv(h, f32(w), ring, b, torch.float32)
            want = torch.cat([ref_u[sl][p0:p0 + n] for sl, p0, n in placed])
            assert (u.double().cpu() - want).abs().max() < 1e-5, (taps, steps, step)
            yy = torch.cat([y[sl][p0:p0 + n] for sl, p0, n in placed])
            parts = torch.stack([yy * 0.25, yy * 0.75]).float().to(DEV)
            ops.scaled_add_norm(h, ops.PartialSum(parts), f32(wn), alpha, eps, ring, b)
            want = torch.cat([ref_x[sl][p0:p0 + n] for sl, p0, n in placed])
            assert (h.double().cpu() - want).abs().max() < 1e-5
            for sl, p0, n in placed:
                at[sl] = p0 + n
        assert at == lens
        assert torch.all(kept[[1, 3]] == 99.0) and torch.all(kept[:, 0] [[1, 3]] == 99.0)      # nobody else's rows were touched
        if taps > 1:
            assert torch.all(kept[[0, 2], 0] == 0)                      # nor the other sublayer's


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


def test_attention_with_head_temperature_and_logarithmic_distance_bias():
    """Random scores, and keys that would win by far placed hundreds of tokens back, at a page's first and last place
    and at the sequence's first token: whether they win depends on the bias r1 ln(1 + r2 n) at exactly that
    distance, with a temperature per head."""
    ops = _ops()
    T, page, H, G, D, V, scale = 700, 16, 6, 2, 24, 40, 0.3
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=F64) for n, d in ((H, D), (G, D), (G, V)))
    temp = 1 + 0.5 * torch.rand(H, generator=g, dtype=F64)
    r1 = torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 0.7], dtype=F64)
    r2 = torch.tensor([1.0, 0.1, 2.0, 0.5, 1.0, 30.0], dtype=F64)
    k[0] = q[650, ::3] * 1.5          # the first token, 650 back
    k[15], k[16] = q[690, ::3] * 1.5, q[691, ::3] * 1.5      # a page's last and first place, hundreds back
    k[640] = q[699, ::3] * 1.5
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 0.05)):
        keys, values, block_table, order = _paged(T, page, G, D, V, dtype, 1)
        for j in range(T):
            keys[order[j // page], :, j % page] = k[j].to(dtype).to(DEV)
            values[order[j // page], :, j % page] = v[j].to(dtype).to(DEV)
        out = torch.zeros(T, H * V, dtype=dtype, device=DEV)
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        f32 = lambda t: t.float().to(DEV).contiguous()
        ops.paged_attention_generic_kv(q.reshape(T, -1).to(dtype).to(DEV), keys, values, _i32(torch.arange(T)), _i32([0] * T),
                                       _i32([1]), block_table, H, G, D, V, page, None, scale, status, out,
                                       head_scale=f32(temp), log_bias=(f32(r1), f32(r2)))
        assert status.tolist() == [0, 0]
        kq, kk, kv = (t.to(dtype).double() for t in (q, k, v))
        ref = pk.biased_attention_core(kq, kk, kv, scale, temp, r1, r2)
        assert (out.double().cpu().view(T, H, V) - ref).abs().max() < tol, dtype
    # the probes matter: without the bias the far keys would take over heads that the bias protects
    flat = pk.biased_attention_core(q, k, v, scale, temp, r1 * 0, r2)
    assert (flat[650] - pk.biased_attention_core(q, k, v, scale, temp, r1, r2)[650]).abs().max() > 0.1


@pytest.mark.parametrize("d,group", [(64, 2), (128, 1), (128, 2), (128, 4)])
def test_tensor_core_attention_with_temperature_and_logarithmic_bias(d, group):
    """The kernels that a bfloat16 run takes at head sizes 64 and 128: a prompt portion that starts in the middle of a
    page with keys before it, and single tokens in the split-key decode kernel; the temperature and the bias are
    evaluated inside them from three numbers per head.  Keys that would win are placed far back."""
    ops = _ops()
    N, past, page, G, scale = 420, 37, 16, 2, 0.2
    H, T = G * group, N - past
    g = torch.Generator().manual_seed(d + group)
    q, k, v = (torch.randn(N, n, d, generator=g, dtype=F64) for n in (H, G, G))
    temp = 1 + 0.5 * torch.rand(H, generator=g, dtype=F64)
    r1, r2 = 1 + 2 * torch.rand(H, generator=g, dtype=F64), 0.1 + 2 * torch.rand(H, generator=g, dtype=F64)
    r1[0] = 0.0
    for i, j in ((419, 0), (418, 15), (300, 16), (200, 3)):
        k[j] = q[i, ::group] * (40.0 / d)          # a score of about ten: wins by far without the bias, loses with it
    q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    ref = pk.biased_attention_core(q[past:], k, v, scale, temp, r1, r2, first_position=past)
    order = np.random.RandomState(2).permutation(N // page + 6)[:-(-N // page)]
    block_table = torch.full((3, len(order) + 2), -1, dtype=torch.int32)
    block_table[1, :len(order)] = torch.as_tensor(order, dtype=torch.int32)
    block_table = block_table.to(DEV)
    cache = torch.zeros(N // page + 6, 2, G, page, d, dtype=torch.bfloat16, device=DEV)
    for j in range(N):
        cache[order[j // page], 0, :, j % page] = k[j].to(torch.bfloat16).to(DEV)
        cache[order[j // page], 1, :, j % page] = v[j].to(torch.bfloat16).to(DEV)
    qd = q[past:].reshape(T, -1).to(torch.bfloat16).to(DEV)
    three = torch.stack([temp, r1, r2], dim=1).float().to(DEV).contiguous()
    out = torch.zeros(T, H * d, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    tiles = _i32([(0, r0) for r0 in range(0, T, ops.PREFILL_TILE_ROWS)])
    ops.paged_attention_prefill_biased(qd, out, 0, cache, tiles, tiles.shape[0], _i32([1]), _i32([0]), _i32([T]), _i32([N]),
                                       block_table, H, G, d, page, None, scale, status, dist_bias_t=three, analytic_bias=True)
    assert status.tolist() == [0, 0]
    assert (out.double().cpu().view(T, H, d) - ref).abs().max() < 0.06
    if ops.prefill_tcgen05_biased_supported(d, page, group):
        # the kernel with accumulators in tensor memory: the bias comes from a table by distance that the softmax
        # threads renew tile by tile (here up to four tiles of 128 keys a row tile, so every table is used again)
        o5 = torch.zeros(T, H * d, dtype=torch.bfloat16, device=DEV)
        ops.paged_attention_prefill_tcgen05_biased(qd, o5, cache, tiles, tiles.shape[0], _i32([1]), _i32([0]), _i32([T]),
                                                   _i32([N]), block_table, H, G, d, page, None, scale, status, three)
        assert status.tolist() == [0, 0]
        assert (o5.double().cpu().view(T, H, d) - ref).abs().max() < 0.06
    if ops.fast_attention_supported(d, group):
        for splits in (1, 3):
            a = torch.zeros(T, H * d, dtype=torch.bfloat16, device=DEV)
            picked = [T - 1, T - 2, 5, 263]
            ops.paged_attention_decode(qd, a, cache, _i32(picked + [-1]), 5, _i32(list(range(past, N))), _i32([0] * T), _i32([1]),
                                       block_table, H, G, d, page, None, scale, splits, status, dist_bias_t=three, analytic_bias=True)
            assert status.tolist() == [0, 0]
            assert (a.double().cpu().view(T, H, d)[picked] - ref[picked]).abs().max() < 0.06, splits
    flat = pk.biased_attention_core(q[past:], k, v, scale, temp, r1 * 0, r2, first_position=past)
    assert (flat[T - 1] - ref[T - 1]).abs().max() > 0.1           # the bias decides what the last query sees


@pytest.mark.parametrize("window,dims", [(None, 8), (1, 8), (7, 4), (64, 8), (65, 0)])
def test_latent_attention_kernels_window_edges_and_rotation(window, dims):
    """The kernels between the projections of a latent attention layer, on projections given as numbers: latents
    normed, the shared key part rotated and both written to the pages, queries rotated and folded through the key
    map, attention over the cached rows, values through the value map.  One cached row is turned towards a late
    query so that it would win by far, and placed just inside and just outside that query's window, at a page's
    last and first place and at the sequence's first token.  Against per-head keys and values made plainly."""
    ops = _ops()
    T, page, H, D, P, V, Q, R, scale, eps, base = 150, 16, 3, 12, 8, 20, 28, 24, 0.3, 1e-5, 300.0
    g = torch.Generator().manual_seed(5)
    dq, dkv = torch.randn(T, Q, generator=g, dtype=F64), torch.randn(T, R + P, generator=g, dtype=F64)
    wq, wkv = 1 + 0.1 * torch.randn(Q, generator=g, dtype=F64), 1 + 0.1 * torch.randn(R, generator=g, dtype=F64)
    uq = torch.randn(H * (D + P), Q, generator=g, dtype=F64) * Q ** -0.5 * 2
    uk, uv = torch.randn(H * D, R, generator=g, dtype=F64) * R ** -0.5, torch.randn(H * V, R, generator=g, dtype=F64) * R ** -0.5
    m = {"heads": H, "dim": D, "rot_dim": P, "vdim": V, "kv_rank": R, "rot": {"base": base, "dims": dims}}

    def plain(dkv_rows):
        cq = pk.rms_norm(dq, wq, eps)
        qh = (cq @ uq.T).view(T, H, D + P)
        qn = qh[..., :D]
        qr = pk.rotate_half(qh[..., D:], range(T), dims, base) if dims else qh[..., D:]
        c = pk.rms_norm(dkv_rows[:, :R], wkv, eps)
        kr = pk.rotate_half(dkv_rows[:, None, R:], range(T), dims, base)[:, 0] if dims else dkv_rows[:, R:]
        kn, vv = (c @ uk.T).view(T, H, D), (c @ uv.T).view(T, H, V)
        s = (torch.einsum("thd,shd->hts", qn, kn) + torch.einsum("thd,sd->hts", qr, kr)) * scale
        i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
        vis = (j <= i) & ((i - j < window) if window else True)
        return pk.softmax_core(s, vv.permute(1, 0, 2), vis).permute(1, 0, 2).reshape(T, H * V), qn

    # a latent row that points where head 0 of a late query looks: W_uk[0]^T qn
    _, qn = plain(dkv)
    probes = [(149, (window or 150) - 1), (148, window or 148), (130, (window or 131) - 1), (141, 141 - 16), (140, 140 - 15), (120, 120)]
    for i, back in probes:
        j = i - back
        if 0 <= j < i:
            dkv[j, :R] = (uk[:D].T @ qn[i, 0]) * 3.0
    ref, _ = plain(dkv)
    for dtype, tol in ((torch.float32, 3e-5), (torch.bfloat16, 0.06)):
        keys, _, block_table, order = _paged(T, page, 1, R + P, 0, dtype, 2)
        f32 = lambda t: t.float().to(DEV).contiguous()
        proj = torch.zeros(T, 5 + Q + R + P, dtype=torch.float32, device=DEV)
        proj[:, 5:5 + Q], proj[:, 5 + Q:] = f32(dq), f32(dkv)
        b = _batch([(1, 0, T)])
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        inv_freq = f32(torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)) if dims else None
        cq = ops.latent_prepare(proj, 5, 5 + Q, Q, R, P, dims, f32(wq), f32(wkv), eps, inv_freq, keys, b, block_table, page,
                                status, dtype)
        q32 = (cq.double().cpu() @ uq.T).float().to(DEV)
        qn_dev, packed = ops.latent_q_split(q32, b.positions, inv_freq, H, D, P, R, dims, dtype)
        folded = torch.bmm(qn_dev.double(), uk.view(H, D, R).to(DEV))                     # [H, T, R]
        packed.view(T, H, R + P)[:, :, :R] = folded.permute(1, 0, 2).to(dtype)
        lat = torch.zeros(T, H * R, dtype=dtype, device=DEV)
        ops.paged_attention_generic_kv(packed, keys, None, b.positions, b.token_entry, b.entry_slot, block_table, H, 1, R + P, R,
                                       page, window, scale, status, lat, values_in_keys=True)
        assert status.tolist() == [0, 0]
        got = torch.einsum("thr,hvr->thv", lat.double().cpu().view(T, H, R), uv.view(H, V, R)).reshape(T, H * V)
        assert (got - ref).abs().max() < tol, (window, dims, dtype)
    if window and window > 1:       # the probes matter: one key further out and the result is another
        wide, _ = plain(dkv)
        window += 1
        wider, _ = plain(dkv)
        assert (wide[148] - wider[148]).abs().max() > 0.05


@pytest.mark.parametrize("H,R,P,window,page", [(3, 64, 16, 40, 16), (16, 64, 0, None, 64), (17, 128, 32, 33, 16),
                                                 (40, 64, 48, 32, 32), (6, 256, 16, 97, 64), (33, 512, 64, 64, 16)])
def test_tensor_core_latent_attention_over_cached_rows(H, R, P, window, page):
    """The bfloat16 kernel in which all heads of a token share the staged rows, alone, on packed queries and cached
    rows given as numbers: a prompt portion that starts in the middle of a page beside single decoded tokens of two
    other requests, pages scattered over the pool, head counts that fill no, one and more than one block of heads.
    For some queries one row is turned towards head 0 so that it would win by far, and sits just inside or just outside
    the window, at a page's last and first place, at the sequence's first token and hundreds of rows back."""
    ops = _ops()
    if not ops.latent_attention_supported(R, P):
        pytest.skip("not a size of the kernel")
    g = torch.Generator().manual_seed(H * 1000 + R + P)
    DK, scale = R + P, 0.9 * (R + P) ** -0.5
    lengths = {0: 333, 1: 70, 2: 1}                         # rows cached per slot, the step's tokens included
    n_pages = {s: -(-n // page) for s, n in lengths.items()}
    pool = sum(n_pages.values()) + 4
    order = np.random.RandomState(R + H).permutation(pool)
    table = torch.full((3, max(n_pages.values()) + 1), -1, dtype=torch.int32)
    rows, at = {}, 0
    for s, n in lengths.items():
        table[s, :n_pages[s]] = torch.as_tensor(order[at:at + n_pages[s]], dtype=torch.int32)
        at += n_pages[s]
        rows[s] = bf16_exact(torch.randn(n, DK, generator=g, dtype=F64))
    portions = [(0, 333 - 150, 150), (1, 69, 1), (2, 0, 1)]
    b = _batch(portions)
    T = b.num_tokens
    q = bf16_exact(torch.randn(T, H, DK, generator=g, dtype=F64))
    w = window or 10 ** 6
    # (token of the portion in slot 0, how far back the row sits that head 0 is drawn to)
    first = 333 - 150
    for tok, back in ((149, w - 1 if window else 320), (148, w if window else 300), (120, 0), (100, (first + 100) % page),
                      (99, (first + 99) % page + 1), (60, first + 60)):
        j = first + tok - back
        if 0 <= j:
            rows[0][j] = bf16_exact(q[tok, 0] * 12.0 / scale / q[tok, 0].pow(2).sum())
    cache = torch.zeros(pool, 1, page, DK, dtype=torch.bfloat16, device=DEV)
    for s, n in lengths.items():
        for j in range(n):
            cache[int(table[s, j // page]), 0, j % page] = rows[s][j].to(torch.bfloat16)
    ref = torch.zeros(T, H, R, dtype=F64)
    t = 0
    for slot, p0, n in portions:
        kv = rows[slot][:p0 + n]
        sc = torch.einsum("thd,sd->hts", q[t:t + n], kv) * scale
        i, j = torch.arange(p0, p0 + n)[:, None], torch.arange(p0 + n)[None, :]
        vis = (j <= i) & (i - j < w)
        ref[t:t + n] = pk.softmax_core(sc, kv[None, :, :R].expand(H, -1, -1), vis).permute(1, 0, 2)
        t += n
    out = torch.full((T, H * R), 7.0, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    ops.latent_attention(q.reshape(T, H * DK).to(torch.bfloat16).to(DEV), cache, b.positions, b.token_entry, b.entry_slot,
                         table.to(DEV), H, R, P, page, window, scale, status, out)
    assert status.tolist() == [0, 0]
    err = ((out.double().cpu().view(T, H, R) - ref).abs() / (1.0 + ref.abs())).max()
    assert err < 0.02, (H, R, P, window, page, float(err))
    # the last token of every request alone, as in decoding: each token's rows are dealt to several CTAs and merged
    b1 = _batch([(0, 332, 1), (1, 69, 1), (2, 0, 1)])
    out1 = torch.full((3, H * R), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.latent_attention(q[149:].reshape(3, H * DK).to(torch.bfloat16).to(DEV), cache, b1.positions, b1.token_entry, b1.entry_slot,
                         table.to(DEV), H, R, P, page, window, scale, status, out1)
    assert status.tolist() == [0, 0]
    err = ((out1.double().cpu().view(3, H, R) - ref[149:]).abs() / (1.0 + ref[149:].abs())).max()
    assert err < 0.02, ("single tokens", H, R, P, window, page, float(err))
    if window:                                              # the row just outside the window must not be seen
        assert (ref[148, 0] - rows[0][333 - 150 + 148 - w][:R]).abs().max() > 0.5


def bf16_exact(x):
    return x.to(torch.bfloat16).to(x.dtype)


def test_gelu_gate_activation():
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    gu = torch.randn(5, 2 * 24, generator=g, dtype=F64) * 3
    ref = pk.gelu_tanh(gu[:, :24]) * gu[:, 24:]
    got = ops.silu_and_mul(gu.float().to(DEV), activation="gelu_tanh")
    assert (got.double().cpu() - ref).abs().max() < 1e-5
    parts = torch.stack([gu * 0.5, gu * 0.5]).float().to(DEV)
    got = ops.silu_and_mul(ops.PartialSum(parts), activation="gelu_tanh")
    assert (got.double().cpu() - ref).abs().max() < 1e-5


def test_paired_product_with_the_gelu_gate():
    """Prompt portions of a bfloat16 run take the paired tensor-core product with the activation in its epilogue."""
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    T, K, inter = 300, 256, 384
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=g) * K ** -0.5 * 2).to(torch.bfloat16)
    both = (x.double() @ w.double().T).to(torch.bfloat16).double()
    ref = pk.gelu_tanh(both[:, :inter]) * both[:, inter:]
    got = ops.linear_silu_mul(x.to(DEV), w.to(DEV), torch.bfloat16, "gelu_tanh")
    assert (got.double().cpu() - ref).abs().max() < 0.03 * max(1.0, float(ref.abs().max()))
