"""The Dumalix design in the engine against the plain implementation: each mechanism alone, prompts against
decoding, portions, unequal batches, reused slots and pages, chunk and page edges, long decoding, generation; and
its kernels alone with inputs made so that a fault shows."""
import json
import subprocess
import sys

import pytest
import torch

import dumalix_tiny as T
from plain import dumalix_plain as DP
from tiny import ROOT, TraceRun, random_prompts

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("dumalix")
    return {name: T.make_folder(tmp, name) for name in T.CONFIGS}


def _load(folder, dtype, **kw):
    import transformer_b200 as tb
    kw.setdefault("max_tokens", 2048)
    return tb.load(folder, dtype=dtype, **kw)


def _tokens(folder, n, seed):
    cfg, _ = DP.read_folder(folder)
    return random_prompts(cfg["vocab"], [n], seed)[0]


def greedy(cfg, tensors, prompt, steps):
    seq, out = list(prompt), []
    for _ in range(steps):
        tok = int(torch.argmax(DP.forward(cfg, tensors, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention", "latent", "dense"])
def test_each_mechanism_alone(name, dtype, folders):
    """One layer of one kind: every position of a prompt that crosses a page border, then six tokens decoded."""
    cfg, tensors = DP.read_folder(folders[name])
    tokens = _tokens(folders[name], 76, 11)
    rows = T.run_cuts(_load(folders[name], dtype), tokens, [70])
    T.check_request(cfg, tensors, tokens, rows, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_decoding_token_by_token(dtype, folders):
    cfg, tensors = DP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 90, 5)
    engine = _load(folders["mixed"], dtype)
    whole = T.run_cuts(engine, tokens, [90])
    single = T.run_cuts(engine, tokens, [])
    T.check_request(cfg, tensors, tokens, whole, dtype, "whole")
    T.check_request(cfg, tensors, tokens, single, dtype, "token by token")
    if dtype == "float32":
        for p in whole:
            assert float((whole[p] - single[p]).abs().max()) < 1e-4, f"position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 3, 57, 64, 2], [63, 1, 64, 2], [5, 130], [128, 2, 2], [1, 1, 2, 100], [39, 1, 40, 2]])
def test_portions_of_a_prompt(cuts, dtype, folders):
    """A prompt fed in portions, down to two tokens (shorter than the convolutions' reach), with cuts at and beside
    page borders and chunk borders: the last inputs of every convolution come from the step before, and chunks are
    counted from the sequence's start, not the portion's."""
    cfg, tensors = DP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 140, 6)
    rows = T.run_cuts(_load(folders["mixed"], dtype), tokens, cuts)
    T.check_request(cfg, tensors, tokens, rows, dtype, f"cuts {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_pieces_by_the_engine(dtype, folders):
    cfg, tensors = DP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 100, 16)
    engine = _load(folders["mixed"], dtype, max_step_tokens=37)
    rows = T.run_cuts(engine, tokens, [95])
    T.check_request(cfg, tensors, tokens, rows, dtype, "pieces")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_equals_each_request_alone(dtype, folders):
    """Prompts of 1, 63, 64 and 130 tokens in one step, then decoded together while the short ones end; in slots
    and pages that an earlier batch has used."""
    cfg, tensors = DP.read_folder(folders["mixed"])
    engine = _load(folders["mixed"], dtype, max_tokens=640)
    engine.use_graphs = False
    lens, extra = [1, 63, 64, 130], [2, 6, 4, 8]
    seqs = [_tokens(folders["mixed"], n + e, 20 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    old = [engine.open() for _ in range(3)]
    engine.step(old, [_tokens(folders["mixed"], n, 40 + n) for n in (100, 70, 129)])
    for s in old:
        engine.close(s)
    slots = [engine.open() for _ in seqs]
    rows = [dict() for _ in seqs]
    lg = engine.step(slots, [s[:n] for s, n in zip(seqs, lens)], [list(range(n)) for n in lens]).cpu()
    at = 0
    for i, n in enumerate(lens):
        for p in range(n):
            rows[i][p] = lg[at + p]
        at += n
    live, step = list(range(len(seqs))), 0
    while live:
        live = [i for i in live if lens[i] + step < len(seqs[i])]
        if not live:
            break
        lg = engine.step([slots[i] for i in live], [[seqs[i][lens[i] + step]] for i in live]).cpu()
        for j, i in enumerate(live):
            rows[i][lens[i] + step] = lg[j]
        step += 1
    engine.check_kernels()
    for i, seq in enumerate(seqs):
        T.check_request(cfg, tensors, seq, rows[i], dtype, f"request {i} in the batch")
    alone = _load(folders["mixed"], dtype)
    for i, seq in enumerate(seqs):
        single = T.run_cuts(alone, seq, [lens[i]])
        tol = 1e-4 if dtype == "float32" else T.BF16_REL_TOL * float(max(r.abs().max() for r in single.values()))
        for p in single:
            assert float((single[p] - rows[i][p]).abs().max()) <= tol, f"request {i}, position {p}"


def test_a_slot_and_its_pages_used_again_hold_nothing_of_their_past(folders):
    engine = _load(folders["mixed"], "float32", max_tokens=256)
    a, b = _tokens(folders["mixed"], 130, 1), _tokens(folders["mixed"], 70, 2)
    fresh = T.run_cuts(_load(folders["mixed"], "float32", max_tokens=256), b, [60])
    T.run_cuts(engine, a, [120])
    again = T.run_cuts(engine, b, [60])
    for p in fresh:
        assert torch.equal(fresh[p], again[p]), f"position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_graphs_past_every_chunk(dtype, folders):
    """Three prompt tokens, then 200 tokens decoded through the replayed step: chunks of 40 begin and end among the
    decoded tokens, pages fill up and new ones begin, the convolutions' inputs are carried 200 times."""
    cfg, tensors = DP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 203, 9)
    engine = _load(folders["mixed"], dtype)
    assert engine.graph_safe
    slot = engine.open()
    rows = {2: engine.step([slot], [tokens[:3]]).cpu()[0]}
    for p in range(3, len(tokens)):
        rows[p] = engine.step([slot], [[tokens[p]]]).cpu()[0].clone()
    engine.check_kernels()
    assert engine._graphs, "the decode steps were not replayed from a graph"
    T.check_request(cfg, tensors, tokens, rows, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_reach_the_tensor_core_kernels(dtype, folders):
    cfg, tensors = DP.read_folder(folders["wide"])
    tokens = _tokens(folders["wide"], 300, 3)
    rows = T.run_cuts(_load(folders["wide"], dtype), tokens, [290])
    T.check_request(cfg, tensors, tokens, rows, dtype, "wide")
    # the same in a batch of unequal prompts, decoded together through graphs
    engine = _load(folders["wide"], dtype)
    slots = [engine.open() for _ in range(3)]
    lens = [200, 65, 290]
    engine.step(slots, [tokens[:n] for n in lens])
    for j in range(6):
        lg = engine.step(slots, [[tokens[n + j]] for n in lens]).cpu()
        tol = 1e-4 if dtype == "float32" else T.BF16_REL_TOL * float(lg.abs().max())
        if lens[2] + j in rows:
            assert float((lg[2] - rows[lens[2] + j]).abs().max()) <= tol, f"decoded token {j} in a batch"
    engine.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_no_fast_kernel_takes(dtype, folders):
    cfg, tensors = DP.read_folder(folders["odd"])
    tokens = _tokens(folders["odd"], 80, 8)
    rows = T.run_cuts(_load(folders["odd"], dtype), tokens, [66, 3])
    T.check_request(cfg, tensors, tokens, rows, dtype, "odd")
    batch = _load(folders["odd"], dtype)
    slots = [batch.open() for _ in range(3)]
    lg = batch.step(slots, [tokens[:5], tokens[:66], tokens[:1]]).cpu()
    tol = 1e-4 if dtype == "float32" else T.BF16_REL_TOL * float(lg.abs().max())
    for i, n in enumerate((5, 66, 1)):
        assert float((lg[i] - rows[n - 1]).abs().max()) <= tol, f"request {i} in a batch"


def test_greedy_generation_through_the_entry_point(folders):
    import transformer_b200 as tb
    cfg, tensors = DP.read_folder(folders["mixed"])
    prompts = [_tokens(folders["mixed"], n, 30 + n) for n in (7, 66, 2)]
    engine = _load(folders["mixed"], "float32")
    got = tb.generate(engine, prompts, max_steps=6, stop_tokens=()).tokens
    assert got == [greedy(cfg, tensors, p, 6) for p in prompts]
    res = tb.generate(_load(folders["mixed"], "bfloat16"), prompts, max_steps=6, stop_tokens=())
    assert [len(t) for t in res.tokens] == [6, 6, 6]


def test_trace_runner_and_command_line(folders, tmp_path):
    cfg, tensors = DP.read_folder(folders["mixed"])
    a, b = _tokens(folders["mixed"], 70, 1), _tokens(folders["mixed"], 9, 2)
    run = TraceRun(folders["mixed"], "float32", str(tmp_path / "out"), 256, record_routing=False)
    run.step(0, [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:8], "want": [7]}])
    run.step(1, [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], end=["b"])
    run.step(2, [{"id": "a", "tokens": a[67:68], "want": [0]}], end=["a"])
    first, second, third = (run.logits(i, cfg["vocab"]) for i in range(3))
    run.close()
    ref_a, ref_b = DP.forward(cfg, tensors, a), DP.forward(cfg, tensors, b)
    for got, want in ((first[0], ref_a[0]), (first[1], ref_a[65]), (first[2], ref_b[7]), (second[0], ref_a[66]),
                      (third[0], ref_a[67])):
        assert float((got.double() - want).abs().max()) <= T.FP32_TOL
    assert second.shape[0] == 1
    out = subprocess.run([sys.executable, "-m", "transformer_b200", "generate", "--model", folders["mixed"],
                          "--prompt", " ".join(map(str, b)), "--max-steps", "4", "--dtype", "float32", "--json"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[-1])["tokens"] == [greedy(cfg, tensors, b, 4)]


def test_random_model_of_the_design_runs(folders):
    """Random weights drawn on the device fill every parameter of the design's plan; the engine steps."""
    import transformer_b200 as tb
    engine = tb.random_model(T.MIXED, seed=3, dtype="bfloat16", max_tokens=512)
    slot = engine.open()
    lg = engine.step([slot], [[1, 2, 3, 4, 5]])
    assert torch.isfinite(lg).all()



def _close(got, want, dtype, label=""):
    """A kernel that computes in float and rounds once at the store: within float noise on the 32-bit path, within
    one rounding of the value itself (2^-8 of its size) on the 16-bit path."""
    got, want = got.double(), want.double()
    allowed = 1e-5 * (1.0 + want.abs()) if dtype == "float32" else 2.0 ** -8 * 1.01 * want.abs() + 1e-3
    bad = (got - want).abs() > allowed
    assert not bool(bad.any()), f"{label}: {int(bad.sum())} entries off, the worst by {float(((got - want).abs() - allowed).max()):.3e}"


# ---- kernels alone, with inputs made so that a fault shows ---------------------------------------------------
def _chunk_attention(dtype, nh, nkvh, dk, dv, chunk, lens_before, lens_new, q_of, kernel="general", splits=1, seed=0,
                     sinks=True, turn=True):
    """Runs a windowed attention kernel with chunks, sinks and turned values over a cache filled by hand with
    shuffled pages; returns (out, plain)."""
    from transformer_b200.csrc import lib
    g = torch.Generator().manual_seed(seed)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    B = len(lens_new)
    total = [a + b for a, b in zip(lens_before, lens_new)]
    n_pages = sum((t + 63) // 64 for t in total) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max((t + 63) // 64 for t in total)
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    kc = torch.randn(n_pages, nkvh, 64, dk, generator=g).to(td)         # garbage where nothing was written
    vc = torch.randn(n_pages, nkvh, 64, dv, generator=g).to(td)
    freqs = 0.7 ** torch.arange(dv // 2, dtype=torch.float64)
    ang = torch.arange(max(total) + 1, dtype=torch.float64)[:, None] * freqs[None, :]
    ocos, osin = torch.cos(ang).float(), torch.sin(ang).float()
    keys, vals = [], []
    for b in range(B):
        k = torch.randn(total[b], nkvh, dk, generator=g)
        k = (k / k.norm(dim=-1, keepdim=True)).to(td)
        v = torch.randn(total[b], nkvh, dv, generator=g).to(td)        # as cached: already turned
        keys.append(k.double())
        vals.append(v.double())
        for pg in range((total[b] + 63) // 64):
            table[b, pg] = perm.pop()
            n = min(64, total[b] - pg * 64)
            kc[table[b, pg], :, :n] = k[pg * 64:pg * 64 + n].transpose(0, 1)
            vc[table[b, pg], :, :n] = v[pg * 64:pg * 64 + n].transpose(0, 1)
    nt = sum(lens_new)
    tq = lib.attention_tile_tokens(nh, nkvh) if kernel == "general" else lib.attention_window_mma_tile_tokens(nh, nkvh)
    tile_seq, tile_t0, tile_nq, tok_pos, at = [], [], [], [], 0
    for b in range(B):
        for off in range(0, lens_new[b], tq):
            tile_seq.append(b); tile_t0.append(at + off); tile_nq.append(min(tq, lens_new[b] - off))
        tok_pos += list(range(lens_before[b], total[b]))
        at += lens_new[b]
    group = nh // nkvh
    width = nh * dk + 8
    z = torch.zeros(nt, width, dtype=td)
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            z[at + i, :nh * dk] = q_of(b, lens_before[b] + i, keys[b], g).reshape(-1).to(td)
        at += lens_new[b]
    sink = (torch.randn(nh, generator=g) * 3.0 + 2.0) if sinks else None
    out = torch.empty(nt, nh, dv, dtype=td, device="cuda")
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    scale = 0.25
    d_z, d_kc, d_vc, d_table = z.cuda(), kc.cuda(), vc.cuda(), table.cuda()
    d_seq, d_t0, d_nq, d_pos = I(tile_seq), I(tile_t0), I(tile_nq), I(tok_pos)
    d_sink = sink.cuda() if sinks else None
    d_cos, d_sin = (ocos.cuda(), osin.cuda()) if turn else (None, None)
    partial = torch.empty(nt, nh, max(splits, 1), dv + 2, device="cuda")
    args = (lib.ptr(d_z), lib.ptr(out), lib.ptr(d_kc), lib.ptr(d_vc), 0, lib.ptr(d_seq), lib.ptr(d_t0), lib.ptr(d_nq),
            lib.ptr(d_pos), lib.ptr(d_table), lib.ptr(partial), len(tile_seq), nt, max_pages, width, width, nh, nkvh, dk,
            dv, splits, 1 << 30, 0, scale, 0.0, chunk, lib.ptr(d_sink), lib.ptr(d_cos), lib.ptr(d_sin))
    if kernel == "general":
        lib.call("tb_attention_window_" + ("f32" if dtype == "float32" else "bf16"), *args)
    else:
        assert lib.try_call("tb_attention_window_mma_bf16", *args), "the tensor-core kernel refused sizes it is meant to take"
    torch.cuda.synchronize()
    want = torch.zeros(nt, nh, dv, dtype=torch.float64)
    zd = z.double()
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            p = lens_before[b] + i
            js = [j for j in range(p + 1) if DP.chunk_visible(p, j, chunk or None)]
            for h in range(nh):
                q = zd[at + i, h * dk:(h + 1) * dk]
                s = (keys[b][js, h // group] @ q) * scale
                if sinks:
                    s = torch.cat([s, sink[h].double().view(1)])
                w = torch.softmax(s, 0)[:len(js)]
                o = (w @ vals[b][js, h // group]).view(1, 1, dv)
                if turn:
                    o = DP.rotate_adjacent(o, torch.tensor([p]), freqs, sign=-1.0)
                want[at + i, h] = o.view(dv)
        at += lens_new[b]
    return out.cpu().double(), want


CHUNK_EDGES = ("first of the chunk", "last of the chunk before", "page row 63", "page row 64", "far", "itself")


def _chunk_queries(which, nh, nkvh, chunk):
    """Every head of every query asks, with a score far above the rest, for ONE key."""
    def queries(b, p, k, g):
        c0 = (p // chunk) * chunk if chunk else 0
        j = {"first of the chunk": c0, "last of the chunk before": c0 - 1, "page row 63": (p // 64) * 64 - 1,
             "page row 64": (p // 64) * 64, "far": p - 300, "itself": p}[which]
        j = min(max(j, 0), p)
        return (k[j] * 160.0).float().repeat_interleave(nh // nkvh, dim=0)
    return queries


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkvh, dk, dv, chunk", [(2, 1, 32, 16, 64), (6, 2, 24, 40, 65), (3, 3, 16, 16, 0),
                                                     (5, 1, 130, 6, 1), (6, 3, 48, 48, 100), (20, 1, 16, 32, 500)])
def test_chunk_kernel_one_key_that_stands_out_at_every_edge(dtype, nh, nkvh, dk, dv, chunk):
    """One key far above the rest: the first key of the query's chunk, the last of the chunk before (never visible),
    a page's last and first row, a key 300 tokens back (visible only inside a long chunk), the query's own.  A chunk
    that is counted from the step's first token instead of the sequence's, a mask one token off or a page taken for
    another changes the answer.  Sinks between -4 and 8 in the denominator, the output turned back by the query's
    position.  Prompts, portions that continue a sequence, and single decoded tokens; the keys whole and in slices."""
    for which in CHUNK_EDGES:
        for splits in (1, 3):
            got, want = _chunk_attention(dtype, nh, nkvh, dk, dv, chunk, [0, 130, 64, 321, 40], [70, 1, 1, 1, 90],
                                         _chunk_queries(which, nh, nkvh, chunk), splits=splits)
            tol = 1e-4 if dtype == "float32" else 2e-2
            assert float((got - want).abs().max()) <= tol, f"{which}, {splits} slices: {float((got - want).abs().max()):.3e}"


@pytest.mark.parametrize("nh, nkvh, dk, dv, chunk", [(2, 1, 64, 64, 64), (6, 2, 128, 128, 80), (4, 4, 64, 128, 0),
                                                     (8, 2, 48, 48, 1), (3, 1, 32, 96, 130), (32, 2, 32, 32, 40)])
def test_tensor_core_chunk_kernels_at_every_edge(nh, nkvh, dk, dv, chunk):
    for which in CHUNK_EDGES + ("any",):
        q_of = _chunk_queries(which, nh, nkvh, chunk) if which != "any" else \
            (lambda b, p, k, g: torch.randn(nh, dk, generator=g) * 3.0)
        for lens_new, splits in (([70, 3, 65, 2, 200], 1), ([70, 3, 65, 2, 200], 3)):
            got, want = _chunk_attention("bfloat16", nh, nkvh, dk, dv, chunk, [0, 130, 64, 321, 40], lens_new, q_of,
                                         kernel="mma", splits=splits)
            assert float((got - want).abs().max()) <= 2e-2, f"prompt, {which}, {splits} slices"
        for splits in (1, 4):
            got, want = _chunk_attention("bfloat16", nh, nkvh, dk, dv, chunk, [0, 130, 64, 321, 40, 700],
                                         [1, 1, 1, 1, 1, 1], q_of, kernel="mma", splits=splits)
            assert float((got - want).abs().max()) <= 2e-2, f"decode, {which}, {splits} slices"


def test_a_sink_takes_its_share_of_the_softmax():
    """Without a sink the weights of one visible key sum to one; a sink as large as that key's score halves them."""
    got, want = _chunk_attention("float32", 2, 1, 16, 8, 0, [0], [1], lambda b, p, k, g: torch.zeros(2, 16), sinks=False,
                                 turn=False)
    assert float((got - want).abs().max()) < 1e-5
    from transformer_b200.csrc import lib  # noqa: F401
    got2, want2 = _chunk_attention("float32", 2, 1, 16, 8, 0, [0], [1], lambda b, p, k, g: torch.zeros(2, 16), turn=False)
    assert float((got2 - want2).abs().max()) < 1e-5
    assert float((got2.abs() - got.abs()).max()) < 0          # every entry shrank


@pytest.mark.parametrize("kernel, H, rank, rot", [("float32", 3, 48, 8), ("bfloat16", 8, 128, 16), ("mma1", 8, 128, 32),
                                                  ("mma3", 4, 256, 64), ("mma7", 16, 512, 64)])
def test_causal_latent_kernels_reach_the_first_key_and_keys_far_back(kernel, H, rank, rot):
    """The latent attention without a window (the design's form): every head of every query asks, far above the
    rest, for the sequence's first key, for one 300 tokens back among hundreds, and for the keys on both sides of
    a page border; general and tensor-core kernels, the keys whole and in slices, prompts and single tokens."""
    from test_salepel_gpu import _latent_attention
    causal = 1 << 30            # what the part hands the kernels for "no window"
    dtype = kernel if not kernel.startswith("mma") else "bfloat16"
    splits = int(kernel[3:]) if kernel.startswith("mma") else 0

    def keys(b, n, g):
        k = torch.randn(n, rank + rot, generator=g)
        return k / k.norm(dim=1, keepdim=True)

    for which in ("first", "300 back", "page row 63", "page row 64"):
        def queries(b, p, k, g, which=which):
            j = {"first": 0, "300 back": p - 300, "page row 63": (p // 64) * 64 - 1, "page row 64": (p // 64) * 64}[which]
            j = min(max(j, 0), p)
            return (k[j] * 160.0).float().repeat(H, 1)
        got, want = _latent_attention(dtype, H, rank, rot, causal, [0, 390, 64, 700], [70, 1, 1, 2], queries, keys,
                                      splits=splits)
        tol = 1e-4 if dtype == "float32" else 2e-2
        assert float((got - want).abs().max()) <= tol, f"{which}: {float((got - want).abs().max()):.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [48, 50, 320, 4096])
def test_pair_sum_and_two_norms_in_one_kernel(dtype, d):
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(d)
    x0 = torch.randn(7, d, generator=g) * 3.0
    d1, d2 = torch.randn(7, d, generator=g).to(td), torch.randn(7, d, generator=g).to(td)
    w1, w2 = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) - 0.5
    x = x0.clone().cuda()
    y1 = torch.zeros(7, d + 8, dtype=td, device="cuda")          # a pitch of its own
    y2 = torch.zeros(7, d, dtype=td, device="cuda")
    c1, c2, cw1, cw2 = d1.cuda(), d2.cuda(), w1.cuda(), w2.cuda()
    lib.call("tb_pair_add_rmsnorm_" + lib.suffix(td), lib.ptr(x), lib.ptr(c1), lib.ptr(c2), 0, lib.ptr(cw1), lib.ptr(y1),
             d + 8, lib.ptr(cw2), lib.ptr(y2), d, 1e-5, 7, d)
    v = x0.double() + (d1.double() + d2.double())
    assert float((x.cpu().double() - v).abs().max()) < 1e-5
    _close(y1[:, :d].cpu(), DP.rms_norm(v, w1.double(), 1e-5), dtype, "first norm")
    _close(y2.cpu(), DP.rms_norm(v, w2.double(), 1e-5), dtype, "second norm")
    assert float(y1[:, d:].abs().max()) == 0.0
    # gathered rows, one output, no weight: the sum itself, the stream untouched
    rows = torch.tensor([5, 0], dtype=torch.int32, device="cuda")
    before = x.clone()
    lib.call("tb_pair_add_rmsnorm_" + lib.suffix(td), lib.ptr(x), lib.ptr(c1), 0, lib.ptr(rows), 0, lib.ptr(y2), d, 0, 0, 0,
             0.0, 2, d)
    assert torch.equal(x, before)
    want = (before.cpu().double() + d1.double())[[5, 0]]
    _close(y2[:2].cpu(), want, dtype, "gathered rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps, residual", [(1, 1), (2, 0), (3, 1), (4, 1), (5, 0), (16, 1)])
@pytest.mark.parametrize("C, pad, lens, steps", [
    (20, 4, (9, 23, 4), ([1, 7, 2], [2, 1, 1], [1, 1, 1], [5, 14, 0])),
    # channels in groups of 16 bytes and steps of many tokens: the form that slides a window over a tile of tokens,
    # with portions that start inside a tile, one of them a single token
    (48, 8, (75, 150, 30), ([3, 70, 2], [2, 1, 1], [1, 1, 1], [69, 78, 26])),
])
def test_causal_convolution_across_steps_in_a_used_slot(dtype, taps, residual, C, pad, lens, steps):
    """Three sequences in steps of unequal sizes (down to one token, shorter than the taps' reach) in slots whose
    rows held other sequences' inputs before: the same as the convolution of each whole sequence."""
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(n, C, generator=g).to(td) for n in lens]
    state = torch.randn(5, max(taps - 1, 1) * C + 3, generator=g).cuda()
    slots = [3, 0, 4]
    for s in slots:
        state[s].zero_()
    got = [torch.zeros(n, C, dtype=td) for n in lens]
    at = [0, 0, 0]
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    cw = w.cuda()
    for sizes in steps:
        live = [i for i, n in enumerate(sizes) if n]
        u = torch.cat([seqs[i][at[i]:at[i] + sizes[i]] for i in live])
        nt = u.shape[0]
        du = torch.zeros(nt, C + pad, dtype=td, device="cuda")
        du[:, :C] = u.cuda()
        y = torch.zeros(nt, C, dtype=td, device="cuda")
        starts = [0]
        for i in live:
            starts.append(starts[-1] + sizes[i])
        tok_seq = [b for b, i in enumerate(live) for _ in range(sizes[i])]
        d_seq, d_start, d_slots = I(tok_seq), I(starts), I([slots[i] for i in live])
        decode = all(sizes[i] == 1 for i in live)
        lib.call("tb_causal_conv_" + lib.suffix(td), lib.ptr(du), C + pad, lib.ptr(cw), lib.ptr(state), state.stride(0),
                 lib.ptr(y), C, lib.ptr(d_seq), lib.ptr(d_start), lib.ptr(d_slots), nt, len(live), C, taps, residual,
                 1 if decode else 0)
        torch.cuda.synchronize()
        for b, i in enumerate(live):
            got[i][at[i]:at[i] + sizes[i]] = y[starts[b]:starts[b + 1]].cpu()
            at[i] += sizes[i]
    for i, s in enumerate(seqs):
        want = DP.causal_conv(s.double(), w.double()) + (s.double() if residual else 0)
        _close(got[i], want, dtype, f"sequence {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkvh, dk, dv, rdims, taps", [(4, 2, 16, 24, 8, 3), (3, 3, 10, 6, 10, 2), (2, 1, 64, 32, 0, 0),
                                                          (6, 2, 48, 48, 48, 4), (2, 2, 24, 20, 12, 1),
                                                          (5, 1, 256, 130, 64, 5)])
def test_convolution_head_norms_rotations_and_cache_write(dtype, nh, nkvh, dk, dv, rdims, taps):
    """The kernel between the q-k-v product and the attention, in three steps of one sequence (each continues from
    the state the one before left: a step shorter than the taps' reach, a step of many tokens, which takes the form
    that slides over tiles of tokens, and a few more) and with a second sequence beside it that starts inside a tile:
    queries out, keys and values in the page and row of their position.  ``taps`` 0: no convolution; 1: a weight per
    channel."""
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(nh * 100 + dk)
    C = (nh + nkvh) * dk + nkvh * dv
    n_a, n_b = 140, 5
    za, zb = torch.randn(n_a, C, generator=g).to(td), torch.randn(n_b, C, generator=g).to(td)
    conv = torch.randn(C, max(taps, 1), generator=g) * 0.5
    wq, wk = torch.rand(dk, generator=g) + 0.5, torch.rand(dk, generator=g) + 0.5
    temp = torch.rand(nh, generator=g) + 0.5
    rp = max(rdims // 2, 1)
    f = 0.3 ** torch.arange(rp, dtype=torch.float64)
    fv = 0.6 ** torch.arange(dv // 2, dtype=torch.float64)
    pos_all = torch.arange(200, dtype=torch.float64)[:, None]
    cos, sin = torch.cos(pos_all * f).float() * 1.1, torch.sin(pos_all * f).float() * 1.1
    vcos, vsin = torch.cos(pos_all * fv).float(), torch.sin(pos_all * fv).float()
    table = torch.tensor([[3, 1, 4], [2, 0, 0]], dtype=torch.int32)
    kc = torch.zeros(5, nkvh, 64, dk, dtype=td, device="cuda")
    vc = torch.zeros(5, nkvh, 64, dv, dtype=td, device="cuda")
    state = torch.randn(4, max(taps - 1, 1) * C, generator=g).cuda()
    state[1].zero_(); state[2].zero_()
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    d_conv, d_wq, d_wk, d_temp = conv.cuda(), wq.cuda(), wk.cuda(), temp.cuda()
    d_cos, d_sin, d_vcos, d_vsin, d_table = cos.cuda(), sin.cuda(), vcos.cuda(), vsin.cuda(), table.cuda()
    qs = []
    for (lo, hi, with_b) in ((0, 3, False), (3, 133, True), (133, 140, False)):
        z = torch.cat([za[lo:hi]] + ([zb] if with_b else []))
        nt = z.shape[0]
        dz = z.cuda()
        q = torch.zeros(nt, nh * dk, dtype=td, device="cuda")
        lens = [hi - lo] + ([n_b] if with_b else [])
        tok_seq = [b for b, n in enumerate(lens) for _ in range(n)]
        tok_pos = list(range(lo, hi)) + (list(range(n_b)) if with_b else [])
        starts = [0, hi - lo] + ([hi - lo + n_b] if with_b else [])
        d_seq, d_pos, d_start, d_slots = I(tok_seq), I(tok_pos), I(starts), I([2, 1][:len(lens)])
        lib.call("tb_head_prep_" + lib.suffix(td), lib.ptr(dz), C, lib.ptr(d_conv) if taps else 0, lib.ptr(state),
                 state.stride(0), lib.ptr(d_wq), lib.ptr(d_wk), lib.ptr(d_temp), 1e-5, lib.ptr(d_cos), lib.ptr(d_sin),
                 lib.ptr(d_vcos), lib.ptr(d_vsin), lib.ptr(q), lib.ptr(kc), lib.ptr(vc), lib.ptr(d_seq), lib.ptr(d_pos),
                 lib.ptr(d_start), lib.ptr(d_slots), lib.ptr(d_table), 3, nt, nh, nkvh, dk, dv, rdims, max(taps, 1), 0, 0, 0)
        if taps > 1:
            lib.call("tb_conv_roll_" + lib.suffix(td), lib.ptr(dz), C, lib.ptr(state), state.stride(0), lib.ptr(d_start),
                     lib.ptr(d_slots), len(lens), C, taps)
        torch.cuda.synchronize()
        qs.append(q.cpu())
    tol = 1e-5 if dtype == "float32" else 3e-2
    for z, n, row, got_q in ((za, n_a, 0, torch.cat([qs[0], qs[1][:130], qs[2]])), (zb, n_b, 1, qs[1][130:])):
        u = DP.causal_conv(z.double(), conv.double()) if taps else z.double()
        pos = torch.arange(n)
        nq, nk = nh * dk, nkvh * dk
        q = DP.rms_norm(u[:, :nq].view(n, nh, dk), wq.double(), 1e-5) * temp.double()[None, :, None]
        k = DP.rms_norm(u[:, nq:nq + nk].view(n, nkvh, dk), wk.double(), 1e-5)
        v = u[:, nq + nk:].view(n, nkvh, dv)
        if rdims:
            q, k = DP.rotate_adjacent(q, pos, f, 1.1), DP.rotate_adjacent(k, pos, f, 1.1)
        v = DP.rotate_adjacent(v, pos, fv)
        assert float((got_q.double().view(n, nh, dk) - q).abs().max()) <= tol * float(q.abs().max())
        for p in range(n):
            page, r = int(table[row, p // 64]), p % 64
            assert float((kc[page, :, r].cpu().double() - k[p]).abs().max()) <= tol * float(k.abs().max()), f"key {p}"
            assert float((vc[page, :, r].cpu().double() - v[p]).abs().max()) <= tol * float(v.abs().max()), f"value {p}"
