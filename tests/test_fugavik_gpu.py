"""The Fugavik design in the engine against the plain implementation: each mechanism alone, prompts against
decoding, portions, unequal batches, reused slots and pages, the first tokens, long decoding, generation; and its
kernels alone with inputs made so that a fault shows."""
import json
import math
import subprocess
import sys

import pytest
import torch

import fugavik_tiny as T
from plain import fugavik_plain as FP
from tiny import ROOT, TraceRun, random_prompts

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("fugavik")
    return {name: T.make_folder(tmp, name) for name in T.CONFIGS}


def _load(folder, dtype, **kw):
    import transformer_b200 as tb
    kw.setdefault("max_tokens", 2048)
    return tb.load(folder, dtype=dtype, **kw)


def _tokens(folder, n, seed):
    cfg, _ = FP.read_folder(folder)
    return random_prompts(cfg["vocab"], [n], seed)[0]


def greedy(cfg, tensors, prompt, steps):
    seq, out = list(prompt), []
    for _ in range(steps):
        tok = int(torch.argmax(FP.forward(cfg, tensors, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention", "latent", "delta", "dense", "experts"])
def test_each_mechanism_alone(name, dtype, folders):
    """One kind of layer: every position of a prompt that crosses a page border, then six tokens decoded."""
    cfg, tensors = FP.read_folder(folders[name])
    tokens = _tokens(folders[name], 76, 11)
    rows, routes = T.run_cuts(_load(folders[name], dtype), tokens, [70])
    T.check_request(cfg, tensors, tokens, rows, dtype, name, routes)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_decoding_token_by_token(dtype, folders):
    cfg, tensors = FP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 90, 5)
    engine = _load(folders["mixed"], dtype)
    whole, r1 = T.run_cuts(engine, tokens, [90])
    single, r2 = T.run_cuts(engine, tokens, [])
    T.check_request(cfg, tensors, tokens, whole, dtype, "whole", r1)
    T.check_request(cfg, tensors, tokens, single, dtype, "token by token", r2)
    if dtype == "float32":
        for p in whole:
            assert float((whole[p] - single[p]).abs().max()) < 1e-4, f"position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 3, 57, 64, 2], [63, 1, 64, 2], [5, 130], [128, 2, 2], [1, 1, 2, 100]])
def test_portions_of_a_prompt(cuts, dtype, folders):
    """A prompt fed in portions, down to two tokens (shorter than the convolutions' reach), with cuts at and beside
    page borders: the delta rule's state and the convolutions' last inputs come from the step before, and the values
    a layer blends with are those of the same portion."""
    cfg, tensors = FP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 140, 6)
    rows, routes = T.run_cuts(_load(folders["mixed"], dtype), tokens, cuts)
    T.check_request(cfg, tensors, tokens, rows, dtype, f"cuts {cuts}", routes)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_pieces_by_the_engine(dtype, folders):
    """A prompt longer than the engine's scratch memory allows per step runs as pieces of one step."""
    cfg, tensors = FP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 100, 16)
    engine = _load(folders["mixed"], dtype, max_step_tokens=37)
    rows, routes = T.run_cuts(engine, tokens, [95])
    T.check_request(cfg, tensors, tokens, rows, dtype, "pieces", routes)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "no_experts"])
def test_unequal_batch_equals_each_request_alone(name, dtype, folders):
    """Prompts of 1, 63, 64 and 130 tokens in one step, then decoded together while the short ones end; in slots
    and pages that an earlier batch has used."""
    cfg, tensors = FP.read_folder(folders[name])
    engine = _load(folders[name], dtype, max_tokens=640)
    engine.use_graphs = False
    lens, extra = [1, 63, 64, 130], [2, 6, 4, 8]
    seqs = [_tokens(folders[name], n + e, 20 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    old = [engine.open() for _ in range(3)]
    engine.step(old, [_tokens(folders[name], n, 40 + n) for n in (100, 70, 129)])
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
    alone = _load(folders[name], dtype)
    for i, seq in enumerate(seqs):
        single, routes = T.run_cuts(alone, seq, [lens[i]])
        T.check_request(cfg, tensors, seq, single, dtype, f"request {i} alone", routes)
        tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(max(r.abs().max() for r in single.values()))
        far = [p for p in single if float((single[p] - rows[i][p]).abs().max()) > tol]
        # in bfloat16 a token whose two best experts lie within the rounding may go either way with the batch
        allowed = 0 if dtype == "float32" or name == "no_experts" else max(1, len(single) // 25)
        assert len(far) <= allowed, f"request {i}: positions {far} differ between the batch and the request alone"


def test_a_slot_and_its_pages_used_again_hold_nothing_of_their_past(folders):
    engine = _load(folders["mixed"], "float32", max_tokens=256)
    a, b = _tokens(folders["mixed"], 130, 1), _tokens(folders["mixed"], 70, 2)
    fresh, _ = T.run_cuts(_load(folders["mixed"], "float32", max_tokens=256), b, [60])
    T.run_cuts(engine, a, [120])
    again, _ = T.run_cuts(engine, b, [60])
    for p in fresh:
        assert torch.equal(fresh[p], again[p]), f"position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(dtype, folders):
    """Sequences of one, two and three tokens, alone and side by side: the softmax of the first token holds one key
    and the sink, the convolutions reach before the start, the delta rule reads an empty state."""
    cfg, tensors = FP.read_folder(folders["mixed"])
    engine = _load(folders["mixed"], dtype)
    engine.use_graphs = False
    seqs = [_tokens(folders["mixed"], n, 70 + n) for n in (1, 2, 3)]
    slots = [engine.open() for _ in seqs]
    rec = T.Recorder(engine)
    lg = engine.step(slots, seqs, [list(range(len(s))) for s in seqs]).cpu()
    routes, engine.recorder = rec.take(), None
    at = 0
    for s in seqs:
        mine = {l: r[at:at + len(s)] for l, r in routes.items()}
        T.check_request(cfg, tensors, s, {p: lg[at + p] for p in range(len(s))}, dtype, f"a sequence of {len(s)}", mine)
        at += len(s)


@pytest.mark.parametrize("dtype, name", [("float32", "mixed"), ("bfloat16", "no_experts"), ("float32", "no_experts")])
def test_long_decoding_through_graphs(dtype, name, folders):
    """Three prompt tokens, then 200 tokens decoded through the replayed step: pages fill up and new ones begin, the
    delta rule's state is carried 200 times, the blended values are those of the step at hand."""
    cfg, tensors = FP.read_folder(folders[name])
    tokens = _tokens(folders[name], 203, 9)
    engine = _load(folders[name], dtype)
    assert engine.graph_safe
    slot = engine.open()
    rows = {2: engine.step([slot], [tokens[:3]]).cpu()[0]}
    for p in range(3, len(tokens)):
        rows[p] = engine.step([slot], [[tokens[p]]]).cpu()[0].clone()
    engine.check_kernels()
    assert engine._graphs, "the decode steps were not replayed from a graph"
    T.check_request(cfg, tensors, tokens, rows, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_reach_the_vector_and_tensor_core_kernels(dtype, folders):
    cfg, tensors = FP.read_folder(folders["wide"])
    tokens = _tokens(folders["wide"], 300, 3)
    rows, routes = T.run_cuts(_load(folders["wide"], dtype), tokens, [290])
    T.check_request(cfg, tensors, tokens, rows, dtype, "wide", routes)
    # the same in a batch of unequal prompts, decoded together through graphs
    engine = _load(folders["wide"], dtype)
    slots = [engine.open() for _ in range(3)]
    lens = [200, 65, 290]
    engine.step(slots, [tokens[:n] for n in lens])
    for j in range(6):
        lg = engine.step(slots, [[tokens[n + j]] for n in lens]).cpu()
        tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(lg.abs().max())
        if lens[2] + j in rows:
            assert float((lg[2] - rows[lens[2] + j]).abs().max()) <= tol, f"decoded token {j} in a batch"
    engine.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_no_fast_kernel_takes(dtype, folders):
    cfg, tensors = FP.read_folder(folders["odd"])
    tokens = _tokens(folders["odd"], 80, 8)
    rows, routes = T.run_cuts(_load(folders["odd"], dtype), tokens, [66, 3])
    T.check_request(cfg, tensors, tokens, rows, dtype, "odd", routes)
    batch = _load(folders["odd"], dtype)
    slots = [batch.open() for _ in range(3)]
    lg = batch.step(slots, [tokens[:5], tokens[:66], tokens[:1]]).cpu()
    tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(lg.abs().max())
    for i, n in enumerate((5, 66, 1)):
        assert float((lg[i] - rows[n - 1]).abs().max()) <= tol, f"request {i} in a batch"


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Layers of every kind in an order drawn at random, sizes drawn at random (two of three draws take sizes that
    reach the vector and tensor-core forms): a prompt across several pages and twelve decoded tokens."""
    import random
    rng = random.Random(1000 + seed)
    cfg = T.random_config(rng, nice=seed % 3 != 2)
    folder = T.make_folder(tmp_path, f"drawn{seed}", cfg=cfg, seed=seed)
    cfg, tensors = FP.read_folder(folder)
    n = rng.randrange(150, 330)
    tokens = random_prompts(cfg["vocab"], [n + 12], seed)[0]
    for dtype in DTYPES:
        rows, routes = T.run_cuts(_load(folder, dtype), tokens, [n])
        kinds = " ".join(l["type"][0] + (l["mlp"]["kind"][0] if l["mlp"] else "-") for l in cfg["layers"])
        T.check_request(cfg, tensors, tokens, rows, dtype, f"drawn {seed} ({kinds}, width {cfg['width']})", routes,
                        floor=True)


def test_random_weights_on_the_device_equal_the_written_folder(tmp_path):
    """``tb.random_model`` (weights filled on the device) and ``tb.write_random_model`` + ``tb.load`` give the same
    model: the same logits bit for bit."""
    import transformer_b200 as tb
    cfg = T.CONFIGS["mixed"][0]
    folder = tb.write_random_model(str(tmp_path / "written"), cfg, seed=5, std=0.1)
    tokens = random_prompts(cfg["vocab"], [70], 1)[0]
    a = tb.load(folder, dtype="bfloat16", max_tokens=512)
    b = tb.random_model(cfg, seed=5, dtype="bfloat16", max_tokens=512, std=0.1)
    la = a.step([a.open()], [tokens], [list(range(70))]).cpu()
    lb = b.step([b.open()], [tokens], [list(range(70))]).cpu()
    assert torch.equal(la, lb)


def test_greedy_generation_through_the_entry_point(folders):
    import transformer_b200 as tb
    cfg, tensors = FP.read_folder(folders["mixed"])
    prompts = [_tokens(folders["mixed"], n, 30 + n) for n in (7, 66, 2)]
    engine = _load(folders["mixed"], "float32")
    got = tb.generate(engine, prompts, max_steps=6, stop_tokens=()).tokens
    assert got == [greedy(cfg, tensors, p, 6) for p in prompts]
    res = tb.generate(_load(folders["mixed"], "bfloat16"), prompts, max_steps=6, stop_tokens=())
    assert [len(t) for t in res.tokens] == [6, 6, 6]


def test_trace_runner_and_command_line(folders, tmp_path):
    cfg, tensors = FP.read_folder(folders["mixed"])
    a, b = _tokens(folders["mixed"], 70, 1), _tokens(folders["mixed"], 9, 2)
    run = TraceRun(folders["mixed"], "float32", str(tmp_path / "out"), 256, record_routing=False)
    run.step(0, [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:8], "want": [7]}])
    run.step(1, [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], end=["b"])
    run.step(2, [{"id": "a", "tokens": a[67:68], "want": [0]}], end=["a"])
    first, second, third = (run.logits(i, cfg["vocab"]) for i in range(3))
    run.close()
    ref_a, ref_b = FP.forward(cfg, tensors, a), FP.forward(cfg, tensors, b)
    for got, want in ((first[0], ref_a[0]), (first[1], ref_a[65]), (first[2], ref_b[7]), (second[0], ref_a[66]),
                      (third[0], ref_a[67])):
        assert float((got.double() - want).abs().max()) <= T.FP32_TOL
    assert second.shape[0] == 1
    out = subprocess.run([sys.executable, "-m", "transformer_b200", "generate", "--model", folders["mixed"],
                          "--prompt", " ".join(map(str, b)), "--max-steps", "4", "--dtype", "float32", "--json"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[-1])["tokens"] == [greedy(cfg, tensors, b, 4)]


# ---- kernels alone, with inputs made so that a fault shows ---------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_kernel_in_all_its_forms(dtype):
    """x += N(delta) (a layer norm or an RMS norm of the part's output, or none), y = LN(x) or the sum itself or
    nothing; the delta a tensor or experts' rows summed with weights or without; rows gathered or all."""
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    sfx = "f32" if dtype == "float32" else "bf16"
    tol = 1e-5 if dtype == "float32" else 2e-2

    def norm(u, w, b, eps, center):
        m = u.mean(1, keepdim=True) if center else 0.0
        y = (u - m) / torch.sqrt(((u - m) ** 2).mean(1, keepdim=True) + eps)
        y = y * w
        return y if b is None else y + b

    for d in (48, 50, 192, 4096, 6008, 13000):
        g = torch.Generator().manual_seed(d)
        n = 6
        x0 = torch.randn(n, d, generator=g) * 2 + 0.5
        delta = (torch.randn(n, d, generator=g) * 3 + 1).to(td)
        pw, pb = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g)
        w, b = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g)
        k = 3
        ey = torch.randn(n * k, d, generator=g).to(td)
        pair_row = torch.randperm(n * k, generator=g).to(torch.int32)
        tw = torch.rand(n, k, generator=g)
        rows = torch.tensor([4, 0, 5], dtype=torch.int32)
        dev = lambda t: None if t is None else t.cuda()
        d_delta, d_pw, d_pb, d_w, d_b, d_ey, d_pr, d_tw, d_rows = map(dev, (delta, pw, pb, w, b, ey, pair_row, tw, rows))
        summed = lambda wts: torch.stack([sum((wts[t, j].double() if wts is not None else 1.0) *
                                              ey[pair_row[t * k + j]].double() for j in range(k)) for t in range(n)])
        cases = [  # (delta kind, post norm?, post center, own norm?, own center, gathered rows)
            ("tensor", True, True, True, True, False), ("tensor", True, True, False, False, False),
            ("tensor", True, True, None, False, False), ("tensor", False, False, True, True, False),
            ("none", False, False, True, True, True), ("none", False, False, True, True, False),
            ("weighted", True, True, True, True, True), ("ones", True, True, False, False, False),
            ("tensor", True, False, True, False, False), ("ones", True, True, True, True, True),
        ]
        for kind, post, pc, own, oc, gathered in cases:
            x = x0.clone().cuda()
            n_out = 3 if gathered else n
            y = torch.full((n_out, d), 7.0, dtype=td, device="cuda") if own is not None else None
            u = {"tensor": delta.double(), "none": None, "weighted": summed(tw), "ones": summed(None)}[kind]
            lib.call("tb_post_add_layernorm_" + sfx, lib.ptr(x), lib.ptr(d_delta) if kind == "tensor" else 0,
                     lib.ptr(d_ey) if kind in ("weighted", "ones") else 0,
                     lib.ptr(d_pr) if kind in ("weighted", "ones") else 0, lib.ptr(d_tw) if kind == "weighted" else 0,
                     k if kind in ("weighted", "ones") else 0, lib.ptr(d_pw) if post else 0,
                     lib.ptr(d_pb) if post and pc else 0, 1e-5, 1 if pc else 0, lib.ptr(d_rows) if gathered else 0,
                     lib.ptr(d_w) if own else 0, lib.ptr(d_b) if own and oc else 0, 1e-5, 1 if oc else 0, lib.ptr(y),
                     n_out, d)
            torch.cuda.synchronize()
            v = x0.double()
            if u is not None:
                v = v + (norm(u, pw.double(), pb.double() if pc else None, 1e-5, pc) if post else u)
            label = f"width {d}, {kind}, post {post}/{pc}, own {own}/{oc}, gathered {gathered}"
            if not gathered:
                assert float((x.cpu().double() - v).abs().max()) < 2e-5, label          # the stream itself is float
            else:
                assert torch.equal(x.cpu(), x0), label                                    # rows gathered: nothing written back
            if own is None:
                continue
            pick = v[rows.long()] if gathered else v
            want = norm(pick, w.double(), b.double() if oc else None, 1e-5, oc) if own else pick
            scale = max(1.0, float(want.abs().max()))
            assert float((y.cpu().double() - want).abs().max()) <= tol * scale, label


def _latent_with_sink(dtype, H, rank, lens_before, lens_new, q_of, sinks, gate, kernel="general", splits=1, seed=0):
    """Runs a latent attention kernel (no rotated part, no window) with sinks and head gates over a cache filled by
    hand with shuffled pages; returns (out [nt, H, rank], plain)."""
    from transformer_b200.csrc import lib
    g = torch.Generator().manual_seed(seed)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    B = len(lens_new)
    total = [a + b for a, b in zip(lens_before, lens_new)]
    n_pages = sum((t + 63) // 64 for t in total) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max((t + 63) // 64 for t in total)
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    cache = torch.randn(n_pages, 64, rank, generator=g).to(td)          # garbage where nothing was written
    keys = []
    for b in range(B):
        k = torch.randn(total[b], rank, generator=g)
        k = (k / k.norm(dim=1, keepdim=True)).to(td)
        keys.append(k.double())
        for pg in range((total[b] + 63) // 64):
            table[b, pg] = perm.pop()
            rows = k[pg * 64:(pg + 1) * 64]
            cache[table[b, pg], :rows.shape[0]] = rows
    nt = sum(lens_new)
    tq = lib.latent_attention_tile_tokens(H)
    tile_seq, tile_t0, tile_nq, tok_pos, at = [], [], [], [], 0
    for b in range(B):
        for off in range(0, lens_new[b], tq):
            tile_seq.append(b); tile_t0.append(at + off); tile_nq.append(min(tq, lens_new[b] - off))
        tok_pos += list(range(lens_before[b], total[b]))
        at += lens_new[b]
    qa = torch.zeros(nt, H, rank, dtype=td)
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            qa[at + i] = q_of(b, lens_before[b] + i, keys[b], g).to(td)
        at += lens_new[b]
    ldg = H + 3                                                         # gate logits behind three entries to skip
    gz = torch.randn(nt, ldg, generator=g).to(td) * 2
    q = torch.zeros(nt, H, 8, dtype=td)                                 # a plain part that the kernel must not read
    out = torch.empty(nt, H, rank, dtype=td, device="cuda")
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    scale, window = 0.25, 1 << 30
    d_qa, d_q, d_cache, d_table, d_gz = qa.cuda(), q.cuda(), cache.cuda(), table.cuda(), gz.cuda()
    d_sinks = sinks.float().cuda() if sinks is not None else None
    d_gate = d_gz[:, 3:] if gate else None
    d_seq, d_t0, d_nq, d_pos = I(tile_seq), I(tile_t0), I(tile_nq), I(tok_pos)
    if kernel == "mma":
        partial = torch.empty(nt, H, max(splits, 1), rank + 2, device="cuda")
        ok = lib.try_call("tb_latent_attention_mma_bf16", lib.ptr(d_qa), lib.ptr(d_q), lib.ptr(out), lib.ptr(partial),
                          lib.ptr(d_cache), lib.ptr(d_seq), lib.ptr(d_t0), lib.ptr(d_nq), lib.ptr(d_pos),
                          lib.ptr(d_table), 0, 0, len(tile_seq), nt, max_pages, H * 8, 8, H, rank, 0, 0, window, splits,
                          scale, lib.ptr(d_sinks), lib.ptr(d_gate), ldg)
        assert ok, "the tensor-core kernel refused sizes it is meant to take"
    else:
        lib.call("tb_latent_attention_" + ("f32" if dtype == "float32" else "bf16"), lib.ptr(d_qa), lib.ptr(d_q),
                 lib.ptr(out), lib.ptr(d_cache), lib.ptr(d_seq), lib.ptr(d_t0), lib.ptr(d_nq), lib.ptr(d_pos),
                 lib.ptr(d_table), 0, 0, len(tile_seq), max_pages, H * 8, 8, 8, H, rank, 0, 0, window, scale,
                 lib.ptr(d_sinks), lib.ptr(d_gate), ldg)
    torch.cuda.synchronize()
    want = torch.zeros(nt, H, rank, dtype=torch.float64)
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            p = lens_before[b] + i
            for h in range(H):
                s = (keys[b][:p + 1] @ qa[at + i, h].double()) * scale
                w = FP.sink_softmax(s, sinks[h]) if sinks is not None else torch.softmax(s, 0)
                o = w @ keys[b][:p + 1]
                want[at + i, h] = o * torch.sigmoid(gz[at + i, 3 + h].double()) if gate else o
        at += lens_new[b]
    return out.cpu().double(), want


LATENT_EDGES = ("first key", "far", "page row 63", "page row 64", "itself", "any")


def _latent_queries(which, H, rank):
    def queries(b, p, k, g):
        if which == "any":
            return torch.randn(H, rank, generator=g) * 8.0
        j = {"first key": 0, "far": p - 300, "page row 63": (p // 64) * 64 - 1, "page row 64": (p // 64) * 64,
             "itself": p}[which]
        j = min(max(j, 0), p)
        return (k[j] * 160.0).float().repeat(H, 1)
    return queries


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, rank", [(2, 32), (5, 24), (20, 64), (1, 130), (3, 11)])
def test_latent_kernel_with_sinks_and_head_gates(dtype, H, rank):
    """One key far above the rest (the sequence's first, one hundreds of tokens back, a page's last and first row,
    the token itself), or none: the sink takes its share of the softmax without adding a value, the gate multiplies
    a whole head.  A sink equal to the score of the one key that stands out halves the answer."""
    g = torch.Generator().manual_seed(H)
    sinks = torch.randn(H, generator=g) * 2.0
    for which in LATENT_EDGES:
        got, want = _latent_with_sink(dtype, H, rank, [0, 130, 64, 321, 40], [70, 1, 1, 1, 90],
                                      _latent_queries(which, H, rank), sinks, True)
        tol = 1e-4 if dtype == "float32" else 2e-2
        assert float((got - want).abs().max()) <= tol, f"{which}: {float((got - want).abs().max()):.3e}"
    if dtype == "float32":
        even = torch.tensor([40.0 if h % 2 else -5.0 for h in range(H)])       # 160 * 0.25 = the standing-out score
        got, want = _latent_with_sink(dtype, H, rank, [321], [1], _latent_queries("far", H, rank), even, False)
        assert float((got - want).abs().max()) <= 1e-3
        free, _ = _latent_with_sink(dtype, H, rank, [321], [1], _latent_queries("far", H, rank), None, False)
        for h in range(H):
            ratio = float(got[0, h].norm() / free[0, h].norm())
            assert abs(ratio - (0.5 if h % 2 else 1.0)) < 1e-2, f"head {h}: the sink took {1 - ratio:.3f} of the softmax"


@pytest.mark.parametrize("splits", [1, 3, 7])
@pytest.mark.parametrize("H, rank", [(2, 32), (5, 96), (20, 64), (16, 128), (3, 160)])
def test_tensor_core_latent_kernel_with_sinks_and_head_gates(H, rank, splits):
    g = torch.Generator().manual_seed(H + rank)
    sinks = torch.randn(H, generator=g) * 2.0
    for which in LATENT_EDGES:
        got, want = _latent_with_sink("bfloat16", H, rank, [0, 130, 64, 321, 40], [70, 1, 1, 1, 90],
                                      _latent_queries(which, H, rank), sinks, True, kernel="mma", splits=splits)
        assert float((got - want).abs().max()) <= 2e-2, f"{which}, {splits} slices: {float((got - want).abs().max()):.3e}"
    # a sink far above every score leaves nothing; one far below changes nothing
    for value, factor in ((200.0, 0.0), (-200.0, 1.0)):
        got, _ = _latent_with_sink("bfloat16", H, rank, [200], [1], _latent_queries("any", H, rank),
                                   torch.full((H,), value), False, kernel="mma", splits=splits)
        free, _ = _latent_with_sink("bfloat16", H, rank, [200], [1], _latent_queries("any", H, rank), None, False,
                                    kernel="mma", splits=splits)
        assert float((got - factor * free).abs().max()) <= 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("G, H, dim, vdim, taps", [(1, 1, 16, 32, 4), (2, 4, 64, 40, 2), (3, 3, 12, 7, 1), (1, 2, 128, 128, 4)])
def test_delta_records_with_one_decay_per_head(dtype, G, H, dim, vdim, taps):
    """The kernel before the scan with one decay per head: every key channel of a head carries the same
    g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b), both read with the pitch of a joined product."""
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(dim + taps)
    nt, C = 9, 2 * G * dim + H * vdim
    ldz = C + 5
    z = torch.randn(nt, ldz, generator=g).to(td)
    conv = torch.randn(C, taps, generator=g) * 0.6
    ba = torch.randn(nt, 2 * H + 1, generator=g) * 2          # [beta | decay | one entry to skip]
    A_log, dt = torch.rand(H, generator=g) * 3 - 2.5, torch.randn(H, generator=g) - 1
    size = lib.delta_state_size(G, H, dim, vdim, taps)
    state = torch.zeros(2, size, device="cuda")
    PER, VP = lib.delta_record_size(dim), lib.delta_value_pitch(vdim)
    DP = (PER - 4) // 3
    rec, vals = torch.empty(nt, H, PER, device="cuda"), torch.empty(nt, H, VP, device="cuda")
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    d_z, d_conv, d_ba, d_A, d_dt = z.cuda(), conv.cuda(), ba.cuda(), A_log.cuda(), dt.cuda()
    d_seq, d_start, d_slots = I([0] * nt), I([0, nt]), I([1])
    lib.call("tb_delta_prep_" + ("f32" if dtype == "float32" else "bf16"), lib.ptr(d_z), ldz, lib.ptr(d_conv),
             lib.ptr(state), lib.ptr(d_ba[:, H:]), lib.ptr(d_dt), lib.ptr(d_A), lib.ptr(d_ba), lib.ptr(rec), lib.ptr(vals),
             lib.ptr(d_seq), lib.ptr(d_start), lib.ptr(d_slots), nt, 1, G, H, dim, vdim, taps, 0, 2 * H + 1, 2 * H + 1, 1)
    torch.cuda.synchronize()
    rec = rec.cpu().double()
    y = FP.silu(FP.causal_conv(z[:, :C].double(), conv.double()))
    for h in range(H):
        kv = h // (H // G)
        want_g = torch.exp(-torch.exp(A_log[h].double()) * FP.softplus(ba[:, H + h].double() + dt[h].double()))
        assert float((rec[:, h, 2 * DP:2 * DP + dim] - want_g[:, None]).abs().max()) < 1e-5, f"head {h}: decay"
        assert float((rec[:, h, 3 * DP] - torch.sigmoid(ba[:, h].double())).abs().max()) < 1e-5, f"head {h}: beta"
        q = FP.unit(y[:, kv * dim:(kv + 1) * dim]) * dim ** -0.5
        k = FP.unit(y[:, G * dim + kv * dim:G * dim + (kv + 1) * dim])
        assert float((rec[:, h, :dim] - q).abs().max()) < 1e-5 and float((rec[:, h, DP:DP + dim] - k).abs().max()) < 1e-5
        v = y[:, 2 * G * dim + h * vdim:2 * G * dim + (h + 1) * vdim]
        assert float((vals.cpu().double()[:, h, :vdim] - v).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_rows_scaled_for_experts_that_weight_what_they_read(dtype):
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    for d in (48, 50):
        g = torch.Generator().manual_seed(d)
        nt, k = 7, 3
        x = torch.randn(nt, d, generator=g).to(td)
        w = torch.rand(nt, k, generator=g)
        pair_row = torch.randperm(nt * k, generator=g).to(torch.int32)
        d_x, d_w, d_pr = x.cuda(), w.cuda(), pair_row.cuda()
        for rows in (d_pr, None):
            out = torch.zeros(nt * k, d, dtype=td, device="cuda")
            lib.call("tb_moe_scaled_rows_" + ("f32" if dtype == "float32" else "bf16"), lib.ptr(d_x), lib.ptr(d_w),
                     lib.ptr(rows), lib.ptr(out), nt * k, d, k)
            torch.cuda.synchronize()
            for p in range(nt * k):
                want = (w.view(-1)[p] * x[p // k].float()).to(td)
                at = int(pair_row[p]) if rows is not None else p
                assert torch.equal(out[at].cpu(), want), f"pair {p}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rule", [0, 2])
def test_layer_norm_kernel_with_a_router_riding_along(dtype, rule):
    """The router of the rows the kernel has just written, as stored: the same experts and weights as the router's own
    kernel gives for those rows, and as torch gives (rule 0: softmax over the kept logits; rule 2: sigmoids)."""
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    sfx = "f32" if dtype == "float32" else "bf16"
    for d, E, k in ((48, 5, 2), (192, 8, 1), (2048, 16, 4), (4096, 3, 3)):
        g = torch.Generator().manual_seed(d + rule)
        n = 7
        x0 = torch.randn(n, d, generator=g)
        delta = (torch.randn(n, d, generator=g) * 2).to(td)
        pw, pb = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g) * 0.3
        wr = (torch.randn(E, d, generator=g) * (3.0 / d ** 0.5)).to(td)
        x, y = x0.clone().cuda(), torch.empty(n, d, dtype=td, device="cuda")
        idx = torch.full((n, k), -1, dtype=torch.int32, device="cuda")
        wts = torch.zeros(n, k, device="cuda")
        d_delta, d_pw, d_pb, d_wr = delta.cuda(), pw.cuda(), pb.cuda(), wr.cuda()
        lib.call("tb_post_add_layernorm_router_" + sfx, lib.ptr(x), lib.ptr(d_delta), 0, 0, 0, 0, lib.ptr(d_pw),
                 lib.ptr(d_pb), 1e-5, 1, 0, 0, 0, 0.0, 0, lib.ptr(y), n, d, lib.ptr(d_wr), 0, lib.ptr(idx), lib.ptr(wts),
                 E, k, rule)
        x2, y2 = x0.clone().cuda(), torch.empty(n, d, dtype=td, device="cuda")
        lib.call("tb_post_add_layernorm_" + sfx, lib.ptr(x2), lib.ptr(d_delta), 0, 0, 0, 0, lib.ptr(d_pw), lib.ptr(d_pb),
                 1e-5, 1, 0, 0, 0, 0.0, 0, lib.ptr(y2), n, d)
        torch.cuda.synchronize()
        assert torch.equal(y, y2) and torch.equal(x, x2)
        z = y.cpu().double() @ wr.double().T
        top = torch.topk(z, k, dim=-1)
        assert torch.equal(idx.cpu().long(), top.indices), f"width {d}"
        want = torch.sigmoid(top.values) if rule == 2 else torch.softmax(top.values, dim=-1)
        assert float((wts.cpu().double() - want).abs().max()) < 1e-5, f"width {d}"


def test_squared_relu_in_the_products_epilogue():
    from transformer_b200.parts.linear import gemm_simt, gemm_skinny
    g = torch.Generator().manual_seed(0)
    for M, K, N in ((3, 64, 40), (8, 2048, 96), (16, 128, 24)):
        a = torch.randn(M, K, generator=g)
        w = torch.randn(N, K, generator=g) / K ** 0.5
        want = torch.relu(a.double() @ w.double().T) ** 2
        out = torch.empty(M, N, device="cuda")
        d_a, d_w = a.cuda(), w.cuda()
        gemm_simt(d_a, d_w, out, out_kind=3)
        assert float((out.cpu().double() - want).abs().max()) < 1e-5 * max(1.0, float(want.abs().max()))
        ab, wb = a.bfloat16(), w.bfloat16()
        want = torch.relu(ab.double() @ wb.double().T) ** 2
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        d_a, d_w = ab.cuda(), wb.cuda()
        assert gemm_skinny(d_a, d_w, out, out_kind=3)
        torch.cuda.synchronize()
        assert float((out.cpu().double() - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())
