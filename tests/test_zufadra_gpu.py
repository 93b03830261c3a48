"""The Zufadra design in the engine against the plain implementation: each mechanism alone, prompts against
decoding, portions, unequal batches, reused slots and pages, window, kept-token and page edges, long decoding,
generation; and its kernels alone with inputs made so that a fault shows."""
import json
import subprocess
import sys

import pytest
import torch

import zufadra_tiny as T
from plain import zufadra_plain as ZP
from tiny import ROOT, TraceRun, random_prompts

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("zufadra")
    return {name: T.make_folder(tmp, name) for name in T.CONFIGS}


def _load(folder, dtype, **kw):
    import transformer_b200 as tb
    kw.setdefault("max_tokens", 2048)
    return tb.load(folder, dtype=dtype, **kw)


def _tokens(folder, n, seed):
    cfg, _ = ZP.read_folder(folder)
    return random_prompts(cfg["vocab"], [n], seed)[0]


def greedy(cfg, tensors, prompt, steps):
    seq, out = list(prompt), []
    for _ in range(steps):
        tok = int(torch.argmax(ZP.forward(cfg, tensors, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention", "delta", "dense"])
def test_each_mechanism_alone(name, dtype, folders):
    """One layer of one kind: every position of a prompt that crosses a page border, then six tokens decoded."""
    cfg, tensors = ZP.read_folder(folders[name])
    tokens = _tokens(folders[name], 76, 11)
    rows = T.run_cuts(_load(folders[name], dtype), tokens, [70])
    T.check_request(cfg, tensors, tokens, rows, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_decoding_token_by_token(dtype, folders):
    cfg, tensors = ZP.read_folder(folders["mixed"])
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
@pytest.mark.parametrize("cuts", [[2, 2, 3, 57, 64, 2], [63, 1, 64, 2], [5, 130], [128, 2, 2], [1, 1, 2, 100]])
def test_portions_of_a_prompt(cuts, dtype, folders):
    """A prompt fed in portions, down to two tokens (shorter than the convolutions' reach), with cuts at and beside
    page borders: the state of the delta rule, the convolutions' last inputs and the token before each portion's
    first one come from the step before."""
    cfg, tensors = ZP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 140, 6)
    rows = T.run_cuts(_load(folders["mixed"], dtype), tokens, cuts)
    T.check_request(cfg, tensors, tokens, rows, dtype, f"cuts {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_pieces_by_the_engine(dtype, folders):
    """A prompt longer than the engine's scratch memory allows per step runs as pieces of one step."""
    cfg, tensors = ZP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 100, 16)
    engine = _load(folders["mixed"], dtype, max_step_tokens=37)
    rows = T.run_cuts(engine, tokens, [95])
    T.check_request(cfg, tensors, tokens, rows, dtype, "pieces")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_equals_each_request_alone(dtype, folders):
    """Prompts of 1, 63, 64 and 130 tokens in one step, then decoded together while the short ones end; in slots
    and pages that an earlier batch has used."""
    cfg, tensors = ZP.read_folder(folders["mixed"])
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
        tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(max(r.abs().max() for r in single.values()))
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
def test_long_decoding_through_graphs_past_every_window(dtype, folders):
    """Three prompt tokens, then 200 tokens decoded through the replayed step: windows of 5 and 70 pass over decoded
    tokens, the kept first tokens stay, pages fill up and new ones begin, the delta rule's state is carried 200 times."""
    cfg, tensors = ZP.read_folder(folders["mixed"])
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
    cfg, tensors = ZP.read_folder(folders["wide"])
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
        tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(lg.abs().max())
        if lens[2] + j in rows:
            assert float((lg[2] - rows[lens[2] + j]).abs().max()) <= tol, f"decoded token {j} in a batch"
    engine.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_no_fast_kernel_takes(dtype, folders):
    cfg, tensors = ZP.read_folder(folders["odd"])
    tokens = _tokens(folders["odd"], 80, 8)
    rows = T.run_cuts(_load(folders["odd"], dtype), tokens, [66, 3])
    T.check_request(cfg, tensors, tokens, rows, dtype, "odd")
    batch = _load(folders["odd"], dtype)
    slots = [batch.open() for _ in range(3)]
    lg = batch.step(slots, [tokens[:5], tokens[:66], tokens[:1]]).cpu()
    tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(lg.abs().max())
    for i, n in enumerate((5, 66, 1)):
        assert float((lg[i] - rows[n - 1]).abs().max()) <= tol, f"request {i} in a batch"


def test_greedy_generation_through_the_entry_point(folders):
    import transformer_b200 as tb
    cfg, tensors = ZP.read_folder(folders["mixed"])
    prompts = [_tokens(folders["mixed"], n, 30 + n) for n in (7, 66, 2)]
    engine = _load(folders["mixed"], "float32")
    got = tb.generate(engine, prompts, max_steps=6, stop_tokens=()).tokens
    assert got == [greedy(cfg, tensors, p, 6) for p in prompts]
    res = tb.generate(_load(folders["mixed"], "bfloat16"), prompts, max_steps=6, stop_tokens=())
    assert [len(t) for t in res.tokens] == [6, 6, 6]


def test_trace_runner_and_command_line(folders, tmp_path):
    cfg, tensors = ZP.read_folder(folders["mixed"])
    a, b = _tokens(folders["mixed"], 70, 1), _tokens(folders["mixed"], 9, 2)
    run = TraceRun(folders["mixed"], "float32", str(tmp_path / "out"), 256, record_routing=False)
    run.step(0, [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:8], "want": [7]}])
    run.step(1, [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], end=["b"])
    run.step(2, [{"id": "a", "tokens": a[67:68], "want": [0]}], end=["a"])
    first, second, third = (run.logits(i, cfg["vocab"]) for i in range(3))
    run.close()
    ref_a, ref_b = ZP.forward(cfg, tensors, a), ZP.forward(cfg, tensors, b)
    for got, want in ((first[0], ref_a[0]), (first[1], ref_a[65]), (first[2], ref_b[7]), (second[0], ref_a[66]),
                      (third[0], ref_a[67])):
        assert float((got.double() - want).abs().max()) <= T.FP32_TOL
    assert second.shape[0] == 1
    out = subprocess.run([sys.executable, "-m", "transformer_b200", "generate", "--model", folders["mixed"],
                          "--prompt", " ".join(map(str, b)), "--max-steps", "4", "--dtype", "float32", "--json"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[-1])["tokens"] == [greedy(cfg, tensors, b, 4)]


def test_the_pair_embedding_in_a_used_slot_and_with_tokens_fed_on_the_device(folders):
    """The token before a step's first one is state of the slot: a slot used before must not remember its last
    sequence, and decode steps whose tokens never reach the host (``device_tokens``) must see the token before."""
    engine = _load(folders["attention"], "float32")
    tokens = _tokens(folders["attention"], 12, 4)
    want = T.run_cuts(_load(folders["attention"], "float32"), tokens, [6])
    T.run_cuts(engine, _tokens(folders["attention"], 9, 5), [9])          # leaves its last token behind
    engine.use_graphs = True
    slot = engine.open()
    engine.step([slot], [tokens[:6]])
    for p in range(6, 12):
        dev = torch.tensor([tokens[p]], dtype=torch.int32, device="cuda")
        lg = engine.step([slot], [[0]], device_tokens=dev).cpu()[0]
        assert float((lg - want[p]).abs().max()) < 1e-4, f"position {p}"
    engine.close(slot)


# ---- kernels alone, with inputs made so that a fault shows ---------------------------------------------------
def _window_attention(dtype, nh, nkvh, dk, dv, window, keep, cap, lens_before, lens_new, q_of, kernel="general",
                      splits=1, seed=0, gate=True):
    """Runs a windowed attention kernel over a cache filled by hand with shuffled pages; returns (out, plain)."""
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
    keys, vals = [], []
    for b in range(B):
        k = torch.randn(total[b], nkvh, dk, generator=g)
        k = (k / k.norm(dim=-1, keepdim=True)).to(td)
        v = torch.randn(total[b], nkvh, dv, generator=g).to(td)
        keys.append(k.double())
        vals.append(v.double())
        for pg in range((total[b] + 63) // 64):
            table[b, pg] = perm.pop()
            n = min(64, total[b] - pg * 64)
            kc[table[b, pg], :, :n] = k[pg * 64:pg * 64 + n].transpose(0, 1)
            vc[table[b, pg], :, :n] = v[pg * 64:pg * 64 + n].transpose(0, 1)
    nt = sum(lens_new)
    tq = lib.attention_tile_tokens(nh, nkvh) if kernel == "general" else lib.attention_window_mma_tile_tokens(nh, nkvh)
    tile_seq, tile_t0, tile_nq, tok_pos, tok_seq, at = [], [], [], [], [], 0
    for b in range(B):
        for off in range(0, lens_new[b], tq):
            tile_seq.append(b); tile_t0.append(at + off); tile_nq.append(min(tq, lens_new[b] - off))
        tok_pos += list(range(lens_before[b], total[b]))
        tok_seq += [b] * lens_new[b]
        at += lens_new[b]
    group = nh // nkvh
    pad = 5 if kernel == "general" else 8            # the tensor-core kernel wants 16-byte aligned rows
    width = nh * dk + pad + nh * dv                  # queries, entries the kernel must skip, the gate
    z = torch.zeros(nt, width, dtype=td)
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            z[at + i, :nh * dk] = q_of(b, lens_before[b] + i, keys[b], g).reshape(-1).to(td)
        at += lens_new[b]
    z[:, nh * dk + pad:] = torch.randn(nt, nh * dv, generator=g).to(td) if gate else 30.0
    out = torch.empty(nt, nh, dv, dtype=td, device="cuda")
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    scale = 0.25
    d_z, d_kc, d_vc, d_table = z.cuda(), kc.cuda(), vc.cuda(), table.cuda()
    d_seq, d_t0, d_nq, d_pos, d_tseq = I(tile_seq), I(tile_t0), I(tile_nq), I(tok_pos), I(tok_seq)
    d_gate = d_z[:, nh * dk + pad:]
    partial = torch.empty(nt, nh, max(splits, 1), dv + 2, device="cuda")
    sfx = "f32" if dtype == "float32" else "bf16"
    if kernel == "general":
        lib.call("tb_attention_window_" + sfx, lib.ptr(d_z), lib.ptr(out), lib.ptr(d_kc), lib.ptr(d_vc), lib.ptr(d_gate),
                 lib.ptr(d_seq), lib.ptr(d_t0), lib.ptr(d_nq), lib.ptr(d_pos), lib.ptr(d_table), lib.ptr(partial),
                 len(tile_seq), nt, max_pages, width, width, nh, nkvh, dk, dv, splits, window, keep, scale, cap, 0, 0, 0, 0)
    else:
        ok = lib.try_call("tb_attention_window_mma_bf16", lib.ptr(d_z), lib.ptr(out), lib.ptr(d_kc), lib.ptr(d_vc),
                          lib.ptr(d_gate), lib.ptr(d_seq), lib.ptr(d_t0), lib.ptr(d_nq), lib.ptr(d_pos),
                          lib.ptr(d_table), lib.ptr(partial), len(tile_seq), nt, max_pages, width, width, nh, nkvh, dk,
                          dv, splits, window, keep, scale, cap, 0, 0, 0, 0)
        assert ok, "the tensor-core kernel refused sizes it is meant to take"
    torch.cuda.synchronize()
    want = torch.zeros(nt, nh, dv, dtype=torch.float64)
    zd = z.double()
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            p = lens_before[b] + i
            js = [j for j in range(p + 1) if ZP.visible(p, j, window, keep)]
            for h in range(nh):
                q = zd[at + i, h * dk:(h + 1) * dk]
                s = (keys[b][js, h // group] @ q) * scale
                if cap:
                    s = cap * torch.tanh(s / cap)
                o = torch.softmax(s, 0) @ vals[b][js, h // group]
                want[at + i, h] = o * torch.sigmoid(zd[at + i, nh * dk + pad + h * dv:nh * dk + pad + (h + 1) * dv])
        at += lens_new[b]
    return out.cpu().double(), want


EDGES = ("oldest inside", "newest outside", "last kept", "first not kept", "page row 63", "page row 64", "far")


def _edge_queries(which, nh, nkvh, window, keep):
    """Every head of every query asks, with a score far above the rest, for ONE key."""
    def queries(b, p, k, g):
        j = {"oldest inside": p - window + 1, "newest outside": p - window, "last kept": keep - 1,
             "first not kept": keep, "page row 63": (p // 64) * 64 - 1, "page row 64": (p // 64) * 64,
             "far": p - 300}[which]
        j = min(max(j, 0), p)
        return (k[j] * 160.0).float().repeat_interleave(nh // nkvh, dim=0)
    return queries


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkvh, dk, dv, window, keep, cap", [
    (2, 1, 32, 16, 64, 3, 0.0), (6, 2, 24, 40, 65, 0, 30.0), (3, 3, 16, 16, 300, 21, 45.0), (5, 1, 130, 6, 1, 1, 0.0),
    (4, 2, 64, 128, 75, 9, 25.0), (20, 1, 16, 32, 10, 70, 10.0)])
def test_window_kernel_one_key_that_stands_out_at_every_edge(dtype, nh, nkvh, dk, dv, window, keep, cap):
    """One key far above the rest: the oldest inside the window, the newest outside it, the last kept first token
    and the first that is not kept, a page's last and first row, a key hundreds of tokens back (visible only if
    kept).  A window or a kept range that is one token off, or a page taken for another, changes the answer from
    that key's value to something else.  Prompts, portions that continue a sequence, and single decoded tokens;
    the key range whole and in slices."""
    for which in EDGES:
        for splits in (1, 3):
            got, want = _window_attention(dtype, nh, nkvh, dk, dv, window, keep, cap, [0, 130, 64, 321, 40],
                                          [70, 1, 1, 1, 90], _edge_queries(which, nh, nkvh, window, keep),
                                          splits=splits)
            tol = 1e-4 if dtype == "float32" else 2e-2
            assert float((got - want).abs().max()) <= tol, f"{which}, {splits} slices: {float((got - want).abs().max()):.3e}"


@pytest.mark.parametrize("nh, nkvh, dk, dv, window, keep, cap", [
    (2, 1, 64, 64, 64, 3, 0.0), (6, 2, 128, 128, 80, 12, 40.0), (4, 4, 64, 128, 300, 0, 30.0), (8, 2, 128, 64, 1, 1, 0.0),
    (3, 1, 32, 96, 130, 70, 10.0), (32, 2, 32, 32, 40, 3, 0.0)])
def test_tensor_core_window_kernels_at_every_edge(nh, nkvh, dk, dv, window, keep, cap):
    """The same questions put to the tensor-core kernel: prompts and portions, and single decoded tokens, with the
    visited pages whole and in slices."""
    for which in EDGES + ("any",):
        q_of = _edge_queries(which, nh, nkvh, window, keep) if which != "any" else \
            (lambda b, p, k, g: torch.randn(nh, dk, generator=g) * 3.0)
        got, want = _window_attention("bfloat16", nh, nkvh, dk, dv, window, keep, cap, [0, 130, 64, 321, 40],
                                      [70, 3, 65, 2, 200], q_of, kernel="mma")
        assert float((got - want).abs().max()) <= 2e-2, f"prompt, {which}: {float((got - want).abs().max()):.3e}"
        got, want = _window_attention("bfloat16", nh, nkvh, dk, dv, window, keep, cap, [0, 130, 64, 321, 40],
                                      [70, 3, 65, 2, 200], q_of, kernel="mma", splits=3)
        assert float((got - want).abs().max()) <= 2e-2, f"prompt in slices, {which}"
        for splits in (1, 4):
            got, want = _window_attention("bfloat16", nh, nkvh, dk, dv, window, keep, cap, [0, 130, 64, 321, 40, 700],
                                          [1, 1, 1, 1, 1, 1], q_of, kernel="mma", splits=splits)
            assert float((got - want).abs().max()) <= 2e-2, f"decode, {which}, {splits} slices"


@pytest.mark.parametrize("G, H, dim, vdim", [(1, 1, 16, 32), (2, 4, 64, 40), (3, 3, 12, 7), (1, 2, 128, 128), (2, 2, 200, 33)])
def test_delta_rule_kernel_keeps_a_token_for_hundreds_of_steps(G, H, dim, vdim):
    """A value is written strongly once (beta = 1, a unit key), nothing is written for 300 tokens (beta = 0, no
    decay), and a later STEP, in a slot whose row held another sequence's state before, asks with that key: the
    answer is the value.  Then random inputs against the plain recurrence, the sequence in two steps."""
    from transformer_b200.csrc import lib
    g = torch.Generator().manual_seed(dim)
    taps = 3
    C = 2 * G * dim + H * vdim
    size = lib.delta_state_size(G, H, dim, vdim, taps)
    state = torch.randn(3, size, generator=g).cuda()         # rows of earlier sequences
    slot = 1
    state[slot].zero_()                                     # what opening the slot does
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")

    def run(qkv, decay, beta):
        # the records the scan reads, per (token, head): q | k | decay (rows padded: 0, 0, 1) | beta, k.q, 0, 0; and v
        n = qkv.shape[0]
        PER, VP = lib.delta_record_size(dim), lib.delta_value_pitch(vdim)
        DP = (PER - 4) // 3
        rec, vals = torch.zeros(n, H, PER), torch.zeros(n, H, VP)
        rec[:, :, 2 * DP:3 * DP] = 1.0
        for h in range(H):
            kv = h // (H // G)
            q, k = qkv[:, kv * dim:(kv + 1) * dim], qkv[:, G * dim + kv * dim:G * dim + (kv + 1) * dim]
            rec[:, h, :dim], rec[:, h, DP:DP + dim] = q, k
            rec[:, h, 2 * DP:2 * DP + dim] = decay[:, h * dim:(h + 1) * dim]
            rec[:, h, 3 * DP], rec[:, h, 3 * DP + 1] = beta[:, h], (q * k).sum(1)
            vals[:, h, :vdim] = qkv[:, 2 * G * dim + h * vdim:2 * G * dim + (h + 1) * vdim]
        out = torch.empty(n, H * vdim, device="cuda")
        # device copies stay in names until the kernel has run: a temporary's memory would be handed to the next one
        d_rec, d_vals, starts, slots = rec.cuda(), vals.cuda(), I([0, n]), I([slot])
        lib.call("tb_delta_scan", lib.ptr(d_rec), lib.ptr(d_vals), lib.ptr(state), lib.ptr(out),
                 lib.ptr(starts), lib.ptr(slots), n, 1, G, H, dim, vdim, taps)
        torch.cuda.synchronize()
        return out.cpu()

    n = 301
    qkv = torch.zeros(n, C)
    qkv[:, :2 * G * dim] = torch.randn(n, 2 * G * dim, generator=g) * 0.1
    value = torch.randn(H * vdim, generator=g)
    key = torch.zeros(G * dim)
    key[[gi * dim + (3 + gi) % dim for gi in range(G)]] = 1.0
    qkv[0, G * dim:2 * G * dim] = key
    qkv[0, 2 * G * dim:] = value
    beta = torch.zeros(n, H)
    beta[0] = 1.0
    run(qkv, torch.ones(n, H * dim), beta)
    ask = torch.zeros(1, C)
    ask[0, :G * dim] = key
    got = run(ask, torch.ones(1, H * dim), torch.zeros(1, H))
    assert float((got[0] - value).abs().max()) < 1e-5

    state[slot].zero_()
    n = 90
    qkv = torch.randn(n, C, generator=g)
    for part in range(2 * G):
        seg = qkv[:, part * dim:(part + 1) * dim]
        seg /= seg.norm(dim=1, keepdim=True)
    decay, beta = torch.rand(n, H * dim, generator=g) * 0.5 + 0.5, torch.rand(n, H, generator=g)
    got = torch.cat([run(qkv[:50], decay[:50], beta[:50]), run(qkv[50:], decay[50:], beta[50:])])
    want = torch.zeros(n, H, vdim, dtype=torch.float64)
    for h in range(H):
        kv = h // (H // G)
        S = torch.zeros(dim, vdim, dtype=torch.float64)
        for t in range(n):
            q, k = qkv[t, kv * dim:(kv + 1) * dim].double(), qkv[t, G * dim + kv * dim:G * dim + (kv + 1) * dim].double()
            v = qkv[t, 2 * G * dim + h * vdim:2 * G * dim + (h + 1) * vdim].double()
            S = decay[t, h * dim:(h + 1) * dim].double()[:, None] * S
            S = S + torch.outer(k, beta[t, h].double() * (v - S.T @ k))
            want[t, h] = S.T @ q
    assert float((got.double() - want.view(n, -1)).abs().max()) < 2e-4


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_sum_without_a_norm(dtype):
    """The weightless norm: x += delta / rms(delta) * w (or x += delta, or nothing), y = the sum rounded once."""
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    sfx = "f32" if dtype == "float32" else "bf16"
    for d in (48, 50, 192, 4096):
        g = torch.Generator().manual_seed(d)
        x0 = torch.randn(5, d, generator=g)
        delta = torch.randn(5, d, generator=g).to(td)
        w = torch.rand(d, generator=g) + 0.5
        x, y = x0.clone().cuda(), torch.empty(5, d, dtype=td, device="cuda")
        dd, dw = delta.cuda(), w.cuda()
        lib.call("tb_post_add_rmsnorm_" + sfx, lib.ptr(x), lib.ptr(dd), 0, 0, 0, 0, lib.ptr(dw), 1e-5, 0, 0, 0.0,
                 lib.ptr(y), 5, d)
        u = delta.double()
        want = x0.double() + u / torch.sqrt((u * u).mean(1, keepdim=True) + 1e-5) * w.double()
        assert float((x.cpu().double() - want).abs().max()) < 1e-5
        assert float((y.cpu().double() - x.cpu().to(td).double()).abs().max()) == 0.0     # the sum, rounded once
        lib.call("tb_add_rmsnorm_" + sfx, lib.ptr(x), lib.ptr(dd), 0, 0, 0, 0, 0, 0, 0.0, lib.ptr(y), 5, d, 0, 0)
        want2 = want.float().double() + u
        assert float((x.cpu().double() - want2).abs().max()) < 1e-5
        assert float((y.cpu().double() - x.cpu().to(td).double()).abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkvh, dk, dv, rdims, half", [(4, 2, 32, 16, 16, 0), (6, 2, 128, 128, 32, 0), (3, 1, 10, 6, 6, 0),
                                                           (2, 2, 16, 24, 0, 0), (5, 5, 24, 8, 24, 0), (2, 1, 16, 16, 8, 1)])
def test_norm_over_the_whole_projection_rotation_and_cache_write(dtype, nh, nkvh, dk, dv, rdims, half):
    """Both forms of the kernel (16-byte accesses where the sizes allow, entry by entry elsewhere): q and k normed over
    ALL their entries at once, the first ``rdims`` entries of every head turned by the token's angles, q back in
    place, k and v into the page and row of the token's position."""
    from transformer_b200.csrc import lib
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(nh * 100 + dk)
    nt, pad = 5, 8
    width = (nh + nkvh) * dk + nkvh * dv + pad
    z = torch.randn(nt, width, generator=g).to(td)
    qw, kw = torch.rand(nh * dk, generator=g) + 0.5, torch.rand(nkvh * dk, generator=g) + 0.5
    pos = [0, 63, 64, 130, 7]
    seq = [0, 1, 2, 3, 4]
    table = torch.tensor([[3, 0, 0], [5, 0, 0], [1, 2, 0], [4, 6, 7], [0, 0, 0]], dtype=torch.int32)
    rp = max(rdims // 2, 1)
    ang = torch.arange(200, dtype=torch.float64)[:, None] * (0.3 ** torch.arange(rp, dtype=torch.float64))[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    kc = torch.zeros(8, nkvh, 64, dk, dtype=td, device="cuda")
    vc = torch.zeros(8, nkvh, 64, dv, dtype=td, device="cuda")
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    d_z, d_qw, d_kw, d_cos, d_sin, d_table, d_seq, d_pos = z.cuda(), qw.cuda(), kw.cuda(), cos.cuda(), sin.cuda(), \
        table.cuda(), I(seq), I(pos)
    lib.call("tb_qknorm_rope_cache_" + ("f32" if dtype == "float32" else "bf16"), lib.ptr(d_z), width, lib.ptr(d_qw),
             lib.ptr(d_kw), 1e-5, lib.ptr(d_seq), lib.ptr(d_pos), lib.ptr(d_table), 3, lib.ptr(d_cos), lib.ptr(d_sin),
             lib.ptr(kc), lib.ptr(vc), nt, nh, nkvh, dk, dv, rdims, half)
    torch.cuda.synchronize()
    zd = z.double()
    nq, nk = nh * dk, nkvh * dk
    tol = 1e-5 if dtype == "float32" else 2e-2
    for t in range(nt):
        q = ZP.rms_norm(zd[t, :nq], qw.double(), 1e-5).view(nh, dk)
        k = ZP.rms_norm(zd[t, nq:nq + nk], kw.double(), 1e-5).view(nkvh, dk)

        def turn(x):
            y = x.clone()
            for i in range(rdims // 2):
                i0, i1 = (i, i + rdims // 2) if half else (2 * i, 2 * i + 1)
                c, s = cos[pos[t], i].double(), sin[pos[t], i].double()
                y[:, i0] = x[:, i0] * c - x[:, i1] * s
                y[:, i1] = x[:, i1] * c + x[:, i0] * s
            return y
        page, r = int(table[t, pos[t] // 64]), pos[t] % 64
        assert float((d_z[t, :nq].cpu().double() - turn(q).reshape(-1)).abs().max()) <= tol
        assert float((kc[page, :, r].cpu().double() - turn(k)).abs().max()) <= tol
        assert torch.equal(vc[page, :, r].cpu(), z[t, nq + nk:nq + nk + nkvh * dv].view(nkvh, dv))
        assert torch.equal(d_z[t, nq:].cpu(), z[t, nq:])          # k, v and what lies behind them stay as they were
