"""The Salepel design in the engine against the plain implementation: each mechanism alone, prompts against
decoding, portions, unequal batches, reused slots and pages, window and page edges, long decoding, generation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import salepel_tiny as T
from plain import salepel_plain as SP
from tiny import ROOT, TraceRun, random_prompts

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("salepel")
    return {name: T.make_folder(tmp, name) for name in T.CONFIGS}


def _load(folder, dtype, **kw):
    import transformer_b200 as tb
    kw.setdefault("max_tokens", 2048)
    return tb.load(folder, dtype=dtype, **kw)


def _tokens(folder, n, seed):
    cfg, _ = SP.read_folder(folder)
    return random_prompts(cfg["vocab"], [n], seed)[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["latent", "memory", "experts"])
def test_each_mechanism_alone(name, dtype, folders):
    """One layer of one kind: every position of a prompt that crosses a page border, then six tokens decoded."""
    cfg, tensors = SP.read_folder(folders[name])
    tokens = _tokens(folders[name], 76, 11)
    rows, routes = T.run_cuts(_load(folders[name], dtype), tokens, [70])
    T.check_request(cfg, tensors, tokens, rows, routes, dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_decoding_token_by_token(dtype, folders):
    cfg, tensors = SP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 90, 5)
    engine = _load(folders["mixed"], dtype)
    whole, r1 = T.run_cuts(engine, tokens, [90])
    single, r2 = T.run_cuts(engine, tokens, [])
    T.check_request(cfg, tensors, tokens, whole, r1, dtype, "whole")
    T.check_request(cfg, tensors, tokens, single, r2, dtype, "token by token")
    if dtype == "float32":
        for p in whole:
            assert float((whole[p] - single[p]).abs().max()) < 1e-4, f"position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 3, 57, 64, 2], [63, 1, 64, 2], [5, 130], [128, 2, 2]])
def test_portions_of_a_prompt(cuts, dtype, folders):
    """A prompt fed in portions, down to two tokens, with cuts at and beside page borders."""
    cfg, tensors = SP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 140, 6)
    rows, routes = T.run_cuts(_load(folders["mixed"], dtype), tokens, cuts)
    T.check_request(cfg, tensors, tokens, rows, routes, dtype, f"cuts {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batch_equals_each_request_alone(dtype, folders):
    """Prompts of 1, 63, 64 and 130 tokens in one step, then decoded together while the short ones end; in slots
    and pages that an earlier batch has used."""
    cfg, tensors = SP.read_folder(folders["mixed"])
    engine = _load(folders["mixed"], dtype, max_tokens=640)
    engine.use_graphs = False
    lens, extra = [1, 63, 64, 130], [2, 6, 4, 8]
    seqs = [_tokens(folders["mixed"], n + e, 20 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    # an earlier batch leaves its traces in the slots, the pages and the per-sequence state
    old = [engine.open() for _ in range(3)]
    engine.step(old, [_tokens(folders["mixed"], n, 40 + n) for n in (100, 70, 129)])
    for s in old:
        engine.close(s)
    rec = T.Routes(engine)
    slots = [engine.open() for _ in seqs]
    rows = [dict() for _ in seqs]
    routes = [[] for _ in seqs]
    lg = engine.step(slots, [s[:n] for s, n in zip(seqs, lens)], [list(range(n)) for n in lens]).cpu()
    rt, at = rec.take(), 0
    for i, n in enumerate(lens):
        for p in range(n):
            rows[i][p] = lg[at + p]
        routes[i].append({l: r[at:at + n] for l, r in rt.items()})
        at += n
    live = list(range(len(seqs)))
    step = 0
    while live:
        live = [i for i in live if lens[i] + step < len(seqs[i])]
        if not live:
            break
        lg = engine.step([slots[i] for i in live], [[seqs[i][lens[i] + step]] for i in live]).cpu()
        rt = rec.take()
        for j, i in enumerate(live):
            rows[i][lens[i] + step] = lg[j]
            routes[i].append({l: r[j:j + 1] for l, r in rt.items()})
        step += 1
    engine.recorder = None
    engine.check_kernels()
    for i, seq in enumerate(seqs):
        r = {l: torch.cat([part[l] for part in routes[i]]) for l in routes[i][0]}
        T.check_request(cfg, tensors, seq, rows[i], r, dtype, f"request {i} in the batch")
    alone = _load(folders["mixed"], dtype)
    for i, seq in enumerate(seqs):
        single, _ = T.run_cuts(alone, seq, [lens[i]])
        tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(max(r.abs().max() for r in single.values()))
        for p in single:
            assert float((single[p] - rows[i][p]).abs().max()) <= tol, f"request {i}, position {p}"


def test_a_slot_and_its_pages_used_again_hold_nothing_of_their_past(folders):
    engine = _load(folders["mixed"], "float32", max_tokens=256)
    a, b = _tokens(folders["mixed"], 130, 1), _tokens(folders["mixed"], 70, 2)
    fresh, _ = T.run_cuts(_load(folders["mixed"], "float32", max_tokens=256), b, [60])
    T.run_cuts(engine, a, [120])
    again, _ = T.run_cuts(engine, b, [60])
    for p in fresh:
        assert torch.equal(fresh[p], again[p]), f"position {p}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_graphs_past_every_window(dtype, folders):
    """Three prompt tokens, then 200 tokens decoded through the replayed step (windows of 3 to 70 pass over decoded
    tokens, pages fill up and new ones begin)."""
    cfg, tensors = SP.read_folder(folders["mixed"])
    tokens = _tokens(folders["mixed"], 203, 9)
    engine = _load(folders["mixed"], dtype)
    assert engine.graph_safe
    slot = engine.open()
    rows = {2: engine.step([slot], [tokens[:3]]).cpu()[0]}
    for p in range(3, len(tokens)):
        rows[p] = engine.step([slot], [[tokens[p]]]).cpu()[0].clone()
    engine.check_kernels()
    assert engine._graphs, "the decode steps were not replayed from a graph"
    routes = None
    if dtype == "bfloat16":         # the experts chosen, from an eager run of the same steps
        _, routes = T.run_cuts(_load(folders["mixed"], dtype), tokens, [3])
    T.check_request(cfg, tensors, tokens, rows, routes, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_reach_the_tensor_core_kernels(dtype, folders):
    cfg, tensors = SP.read_folder(folders["wide"])
    tokens = _tokens(folders["wide"], 300, 3)
    rows, routes = T.run_cuts(_load(folders["wide"], dtype), tokens, [290])
    T.check_request(cfg, tensors, tokens, rows, routes, dtype, "wide")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_no_fast_kernel_takes(dtype, folders):
    cfg, tensors = SP.read_folder(folders["odd"])
    tokens = _tokens(folders["odd"], 80, 8)
    rows, routes = T.run_cuts(_load(folders["odd"], dtype), tokens, [66, 3])
    T.check_request(cfg, tensors, tokens, rows, routes, dtype, "odd")
    batch = _load(folders["odd"], dtype)
    slots = [batch.open() for _ in range(3)]
    lg = batch.step(slots, [tokens[:5], tokens[:66], tokens[:1]]).cpu()
    tol = 1e-4 if dtype == "float32" else 2 * T.BF16_REL_TOL * float(lg.abs().max())
    for i, n in enumerate((5, 66, 1)):
        assert float((lg[i] - rows[n - 1]).abs().max()) <= tol, f"request {i} in a batch"


def test_greedy_generation_through_the_entry_point(folders):
    import transformer_b200 as tb
    cfg, tensors = SP.read_folder(folders["mixed"])
    prompts = [_tokens(folders["mixed"], n, 30 + n) for n in (7, 66, 2)]
    engine = _load(folders["mixed"], "float32")
    got = tb.generate(engine, prompts, max_steps=6, stop_tokens=()).tokens
    want = [SP.greedy_generate(cfg, tensors, p, 6) for p in prompts]
    assert got == want
    engine16 = _load(folders["mixed"], "bfloat16")
    res = tb.generate(engine16, prompts, max_steps=6, stop_tokens=())
    assert [len(t) for t in res.tokens] == [6, 6, 6]


def test_trace_runner_and_command_line(folders, tmp_path):
    cfg, tensors = SP.read_folder(folders["mixed"])
    a, b = _tokens(folders["mixed"], 70, 1), _tokens(folders["mixed"], 9, 2)
    run = TraceRun(folders["mixed"], "float32", str(tmp_path / "out"), 256, record_routing=False)
    run.step(0, [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:8], "want": [7]}])
    run.step(1, [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], end=["b"])
    run.step(2, [{"id": "a", "tokens": a[67:68], "want": [0]}], end=["a"])
    first, second, third = (run.logits(i, cfg["vocab"]) for i in range(3))
    run.close()
    ref_a, ref_b = SP.forward(cfg, tensors, a), SP.forward(cfg, tensors, b)
    for got, want in ((first[0], ref_a[0]), (first[1], ref_a[65]), (first[2], ref_b[7]), (second[0], ref_a[66]),
                      (third[0], ref_a[67])):
        assert float((got.double() - want).abs().max()) <= T.FP32_TOL
    assert second.shape[0] == 1
    out = subprocess.run([sys.executable, "-m", "transformer_b200", "generate", "--model", folders["mixed"],
                          "--prompt", " ".join(map(str, b)), "--max-steps", "4", "--dtype", "float32", "--json"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[-1])["tokens"] == [SP.greedy_generate(cfg, tensors, b, 4)]


# ---- kernels alone, with inputs made so that a fault shows ---------------------------------------------------
def _dev(x, dtype=None):
    return x.to("cuda", dtype) if dtype else x.to("cuda")


def _latent_attention(dtype, H, rank, rot, window, lens_before, lens_new, q_of, c_of, seed=0, splits=0):
    """Runs the attention kernel over a cache filled by hand with shuffled pages; returns (out [nt, H, rank], plain)."""
    from transformer_b200.csrc import lib
    g = torch.Generator().manual_seed(seed)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    DK, B = rank + rot, len(lens_new)
    total = [a + b for a, b in zip(lens_before, lens_new)]
    n_pages = sum((t + 63) // 64 for t in total) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max((t + 63) // 64 for t in total)
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    cache = torch.zeros(n_pages, 64, DK, dtype=td)
    keys = []
    for b in range(B):
        k = c_of(b, total[b], g).to(td)
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
    q = torch.zeros(nt, H, 4 + rot, dtype=td)          # a plain part of 4 entries that the kernel must skip
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            full = q_of(b, lens_before[b] + i, keys[b], g)     # [H, DK], already on the latent's side, unrotated
            qa[at + i] = full[:, :rank].to(td)
            q[at + i, :, 4:] = full[:, rank:].to(td)
        at += lens_new[b]
    out = torch.empty(nt, H, rank, dtype=td, device="cuda")
    ones, zeros = torch.ones(1024, max(rot // 2, 1), device="cuda"), torch.zeros(1024, max(rot // 2, 1), device="cuda")
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    scale = 0.25
    # device copies stay in names until the kernel has run: a temporary's memory would be handed to the next one
    d_qa, d_q, d_cache, d_table = _dev(qa), _dev(q), _dev(cache), _dev(table)
    d_seq, d_t0, d_nq, d_pos = I(tile_seq), I(tile_t0), I(tile_nq), I(tok_pos)
    if splits:          # the tensor-core kernel, its key range in that many slices
        partial = torch.empty(nt, H, splits, rank + 2, device="cuda")
        lib.call("tb_latent_attention_mma_bf16", lib.ptr(d_qa), lib.ptr(d_q), lib.ptr(out), lib.ptr(partial),
                 lib.ptr(d_cache), lib.ptr(d_seq), lib.ptr(d_t0), lib.ptr(d_nq), lib.ptr(d_pos), lib.ptr(d_table),
                 lib.ptr(ones), lib.ptr(zeros), len(tile_seq), nt, max_pages, H * (4 + rot), 4 + rot, H, rank, rot, rot,
                 window, splits, scale, 0, 0, 0)
    else:
        lib.call("tb_latent_attention_" + ("f32" if dtype == "float32" else "bf16"), lib.ptr(d_qa), lib.ptr(d_q),
                 lib.ptr(out), lib.ptr(d_cache), lib.ptr(d_seq), lib.ptr(d_t0), lib.ptr(d_nq), lib.ptr(d_pos),
                 lib.ptr(d_table), lib.ptr(ones), lib.ptr(zeros), len(tile_seq), max_pages, H * (4 + rot), 4 + rot, 4, H,
                 rank, rot, rot, window, scale, 0, 0, 0)
    torch.cuda.synchronize()
    from transformer_b200.csrc.lib import gemm_tc_status
    assert gemm_tc_status() == 0
    want = torch.zeros(nt, H, rank, dtype=torch.float64)
    at = 0
    for b in range(B):
        for i in range(lens_new[b]):
            p = lens_before[b] + i
            lo = max(0, p - window + 1)
            full = torch.cat([qa[at + i].double(), q[at + i, :, 4:].double()], dim=1)
            for h in range(H):
                s = (keys[b][lo:p + 1] @ full[h]) * scale
                want[at + i, h] = torch.softmax(s, 0) @ keys[b][lo:p + 1, :rank]
        at += lens_new[b]
    return out.cpu().double(), want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, rank, rot, window", [(2, 32, 8, 64), (5, 24, 16, 65), (20, 64, 0, 300), (1, 130, 6, 1),
                                                  (2, 256, 16, 50), (1, 512, 64, 20)])
def test_attention_kernel_one_key_that_stands_out_at_every_edge(dtype, H, rank, rot, window):
    """Every head of every query asks, with a score far above the rest, for ONE key: the oldest inside its window,
    the newest outside it, the one at a page's last row or first row, or one hundreds of tokens back.  A window
    that is one token off, or a page taken for another, changes the answer from that key's value to something
    else."""
    def keys(b, n, g):
        k = torch.randn(n, rank + rot, generator=g)
        return k / k.norm(dim=1, keepdim=True)

    for which in ("oldest inside", "newest outside", "page row 63", "page row 64"):
        def queries(b, p, k, g, which=which):
            j = {"oldest inside": p - window + 1, "newest outside": p - window, "page row 63": (p // 64) * 64 - 1,
                 "page row 64": (p // 64) * 64}[which]
            j = min(max(j, 0), p)
            return (k[j] * 160.0).float().repeat(H, 1)
        got, want = _latent_attention(dtype, H, rank, rot, window, [0, 130, 64, 321], [70, 1, 1, 1], queries, keys)
        tol = 1e-4 if dtype == "float32" else 2e-2
        assert float((got - want).abs().max()) <= tol, f"{which}: {float((got - want).abs().max()):.3e}"


@pytest.mark.parametrize("splits", [1, 3, 7])
@pytest.mark.parametrize("H, rank, rot, window", [(2, 32, 16, 64), (5, 96, 16, 65), (20, 64, 0, 300), (16, 128, 32, 1),
                                                  (16, 256, 32, 100), (16, 512, 64, 70), (3, 160, 16, 40),
                                                  (2, 288, 16, 30)])
def test_tensor_core_attention_kernel_at_every_edge(H, rank, rot, window, splits):
    """The same questions put to the tensor-core kernel, with the key range whole and in slices."""
    def keys(b, n, g):
        k = torch.randn(n, rank + rot, generator=g)
        return k / k.norm(dim=1, keepdim=True)

    for which in ("oldest inside", "newest outside", "page row 63", "page row 64", "any"):
        def queries(b, p, k, g, which=which):
            if which == "any":
                return torch.randn(H, rank + rot, generator=g) * 3.0
            j = {"oldest inside": p - window + 1, "newest outside": p - window, "page row 63": (p // 64) * 64 - 1,
                 "page row 64": (p // 64) * 64}[which]
            j = min(max(j, 0), p)
            return (k[j] * 160.0).float().repeat(H, 1)
        got, want = _latent_attention("bfloat16", H, rank, rot, window, [0, 130, 64, 321], [70, 1, 1, 1], queries, keys,
                                      splits=splits)
        assert float((got - want).abs().max()) <= 2e-2, f"{which}: {float((got - want).abs().max()):.3e}"


@pytest.mark.parametrize("kernel", ["scan", "chunk"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, dim, vdim", [(2, 16, 24), (1, 40, 70), (3, 128, 33), (2, 64, 64), (1, 256, 32)])
def test_matrix_memory_kernel_keeps_a_token_for_hundreds_of_steps(dtype, H, dim, vdim, kernel):
    """Gates made so that one early token is written at full strength and (almost) nothing is forgotten: asked with
    that token's key hundreds of tokens later, in a later step and in a slot used before, the answer is its value."""
    from transformer_b200.csrc import lib
    g = torch.Generator().manual_seed(4)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    lens = [300, 7]
    nt, B, cap = sum(lens) , 2, 30.0
    ld = 2 * H * dim + H * vdim
    qkv = (torch.randn(nt + B, ld, generator=g) * 0.5).to(td)
    gates = torch.cat([torch.randn(nt + B, H, generator=g) - 6.0, torch.full((nt + B, H), 12.0)], dim=1)
    special = {0: 5, 1: 2}                                   # sequence -> the token that is written strongly
    starts = [0, lens[0]]
    for b, j in special.items():
        gates[starts[b] + j, :H] = 6.0
    # the last token of each sequence comes in a step of its own and asks with the special token's key
    for b in range(B):
        qkv[nt + b, :H * dim] = qkv[starts[b] + special[b], H * dim:2 * H * dim] * 4.0
        gates[nt + b, :H] = -20.0
    bias = torch.zeros(2 * H)
    size = lib.mlstm_state_size(dim, vdim)
    state = torch.randn(4, H, size, device="cuda")           # slots 3 and 1 are used: what they held must not matter
    slots = torch.tensor([3, 1], dtype=torch.int32, device="cuda")
    state[3].zero_(); state[1].zero_()
    out = torch.empty(nt + B, H * vdim, device="cuda")
    sfx = "f32" if dtype == "float32" else "bf16"
    I = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    dq, dg, db, starts1, starts2 = _dev(qkv), _dev(gates), _dev(bias), I([0, lens[0], nt]), I([0, 1, 2])
    # the prompts token by token or 64 tokens at a time (300 = four chunks and a part of one); the last token alone
    lib.call(f"tb_mlstm_{kernel}_" + sfx, lib.ptr(dq), lib.ptr(dg), lib.ptr(db), lib.ptr(state), lib.ptr(out),
             lib.ptr(starts1), lib.ptr(slots), B, ld, H, dim, vdim, cap, dim ** -0.5)
    lib.call("tb_mlstm_scan_" + sfx, lib.ptr(dq[nt:]), lib.ptr(dg[nt:]), lib.ptr(db), lib.ptr(state),
             lib.ptr(out[nt:]), lib.ptr(starts2), lib.ptr(slots), B, ld, H, dim, vdim, cap, dim ** -0.5)
    torch.cuda.synchronize()
    got = out.cpu().double()
    x = qkv.double()
    for b in range(B):
        idx = list(range(starts[b], starts[b] + lens[b])) + [nt + b]
        ig = cap * torch.tanh(gates[idx, :H].double() / cap)
        fg = torch.nn.functional.logsigmoid(cap * torch.tanh(gates[idx, H:].double() / cap))
        for h in range(H):
            S, n, m = torch.zeros(dim, vdim, dtype=torch.float64), torch.zeros(dim, dtype=torch.float64), 0.0
            for t, row in enumerate(idx):
                q = x[row, h * dim:(h + 1) * dim] * dim ** -0.5
                k = x[row, (H + h) * dim:(H + h + 1) * dim]
                v = x[row, 2 * H * dim + h * vdim:2 * H * dim + (h + 1) * vdim]
                m_new = max(float(fg[t, h]) + m, float(ig[t, h]))
                keep, take = np.exp(float(fg[t, h]) + m - m_new), np.exp(float(ig[t, h]) - m_new)
                S, n, m = keep * S + take * torch.outer(k, v), keep * n + take * k, m_new
                want = (S.T @ q) / (max(abs(float(n @ q)), np.exp(-m)) + 1e-6)
                diff = float((got[row, h * vdim:(h + 1) * vdim] - want).abs().max())
                assert diff <= 2e-4 * max(1.0, float(want.abs().max())), f"sequence {b}, head {h}, token {t}: {diff:.3e}"
            # the question of the last step is answered with the special token's value, to a few percent
            v_special = x[starts[b] + special[b], 2 * H * dim + h * vdim:2 * H * dim + (h + 1) * vdim]
            last = got[nt + b, h * vdim:(h + 1) * vdim]
            cos = float(last @ v_special / (last.norm() * v_special.norm()))
            assert cos > 0.97, f"sequence {b}, head {h}: the early token is lost (cosine {cos:.3f})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_of_a_delta_then_sum_then_norm(dtype):
    from transformer_b200.csrc import lib
    g = torch.Generator().manual_seed(0)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    nt, d, k = 9, 200, 3
    x = torch.randn(nt, d, generator=g)
    delta = (torch.randn(nt, d, generator=g) * 3).to(td)
    wy = torch.randn(nt * k, d, generator=g).to(td)
    idx = torch.randperm(nt * k, generator=g).to(torch.int32)
    wts = torch.rand(nt, k, generator=g)
    pw, w = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    sfx = "f32" if dtype == "float32" else "bf16"
    norm = lambda u, wt, eps: u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * wt
    d_wy, d_idx, d_wts, d_delta, d_pw, d_w = _dev(wy), _dev(idx), _dev(wts), _dev(delta), _dev(pw), _dev(w)
    for weighted in (False, True):
        xd, y = _dev(x.clone()), torch.empty(nt, d, dtype=td, device="cuda")
        args = (0, lib.ptr(d_wy), lib.ptr(d_idx), lib.ptr(d_wts), k) if weighted else (lib.ptr(d_delta), 0, 0, 0, 0)
        lib.call("tb_post_add_rmsnorm_" + sfx, lib.ptr(xd), *args, lib.ptr(d_pw), 1e-5, 0, lib.ptr(d_w), 1e-6,
                 lib.ptr(y), nt, d)
        torch.cuda.synchronize()
        u = (wts.double()[:, :, None] * wy.double()[idx.long()].view(nt, k, d)).sum(1) if weighted else delta.double()
        v = x.double() + norm(u, pw.double(), 1e-5)
        assert float((xd.cpu().double() - v).abs().max()) < 1e-5
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert float((y.cpu().double() - norm(v, w.double(), 1e-6)).abs().max()) < tol


def test_scored_router_and_pass_through_rows():
    from transformer_b200.csrc import lib
    g = torch.Generator().manual_seed(2)
    nt, d, E, ident, k = 40, 64, 5, 3, 3
    R = E + ident
    x = torch.randn(nt, d, generator=g)
    wr = torch.randn(R, d, generator=g) * 0.3
    bias = torch.randn(R, generator=g) * 0.2
    idx = torch.empty(nt, k, dtype=torch.int32, device="cuda")
    w = torch.empty(nt, k, device="cuda")
    offsets = torch.empty(R + 1, dtype=torch.int32, device="cuda")
    sorted_token = torch.empty(nt * k, dtype=torch.int32, device="cuda")
    pair_row = torch.empty(nt * k, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    xd, d_wr, d_bias = _dev(x), _dev(wr), _dev(bias)
    lib.call("tb_router_scored_f32", lib.ptr(xd), lib.ptr(d_wr), lib.ptr(d_bias), lib.ptr(idx), lib.ptr(w),
             lib.ptr(offsets), lib.ptr(sorted_token), lib.ptr(pair_row), lib.ptr(done), nt, d, R, k)
    want_idx, want_w, _ = SP.route(x.double(), {"router": wr.double(), "correction": bias.double()}, k)
    assert idx.cpu().long().tolist() == want_idx.tolist()
    assert float((w.cpu().double() - want_w).abs().max()) < 1e-6
    off = offsets.cpu().tolist()
    assert off[0] == 0 and off[-1] == nt * k and int(done.item()) == 0
    y = torch.full((nt * k, d), -7.0, device="cuda")
    lib.call("tb_moe_identity_rows_f32", lib.ptr(xd), lib.ptr(y), lib.ptr(offsets), lib.ptr(sorted_token), 0, 1, nt * k,
             d, E)
    y, pr = y.cpu(), pair_row.cpu().long()
    for t in range(nt):
        for j in range(k):
            row = y[pr[t * k + j]]
            assert torch.equal(row, x[t]) if int(want_idx[t, j]) >= E else bool((row == -7.0).all())
    y2 = torch.full((nt * k, d), -7.0, device="cuda")
    lib.call("tb_moe_identity_rows_f32", lib.ptr(xd), lib.ptr(y2), 0, 0, lib.ptr(idx), k, nt * k, d, E)
    for p in range(nt * k):
        assert torch.equal(y2[p].cpu(), x[p // k]) if int(want_idx.view(-1)[p]) >= E else bool((y2[p] == -7.0).all())


@pytest.mark.parametrize("rows", [6, 40, 700])
def test_clamped_gate_in_every_product_kernel(rows):
    """The (gate, up) pair with limits below what the products reach, so that every clamp is at work."""
    from transformer_b200.parts.linear import grouped_matmul
    g = torch.Generator().manual_seed(rows)
    G, K, N, alpha, limit = 3, 64, 48, 1.702, 0.8
    x = torch.randn(rows, K, generator=g)
    w = torch.randn(G, 2 * N, K, generator=g) * 0.3
    cuts = sorted(torch.randint(0, rows + 1, (G - 1,), generator=g).tolist())
    offsets = torch.tensor([0] + cuts + [rows], dtype=torch.int32)
    for td, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        xs, ws = x.to(td), w.to(td)
        out = torch.empty(rows, N, dtype=td, device="cuda")
        ws_d, xs_d, off_d = _dev(ws), _dev(xs), _dev(offsets)
        grouped_matmul(xs_d, ws_d, out, group_offsets=off_d, groups=G, swiglu=True, max_group_rows=rows,
                       glu=(alpha, limit))
        torch.cuda.synchronize()
        for gi in range(G):
            lo, hi = int(offsets[gi]), int(offsets[gi + 1])
            z = xs[lo:hi].double() @ ws[gi].double().T
            gate, up = z[:, :N].clamp(max=limit), z[:, N:].clamp(-limit, limit)
            want = gate * torch.sigmoid(alpha * gate) * (up + 1)
            if hi > lo:
                assert float((out[lo:hi].cpu().double() - want).abs().max()) < tol, (td, gi)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M, K", [(3, 24), (100, 24), (8, 64), (16, 128)])
def test_products_batched_over_heads_with_pitches(dtype, M, K):
    from transformer_b200.parts.linear import batched_matmul
    g = torch.Generator().manual_seed(M)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    H, N, pad = 5, 40, 8
    a = torch.randn(M, H, K + pad, generator=g).to(td)
    w = (torch.randn(H, N, K, generator=g) * 0.3).to(td)
    out = torch.zeros(M, H, N, dtype=td, device="cuda")
    a_d, w_d = _dev(a), _dev(w)
    batched_matmul(a_d[:, :, :K], w_d, out)
    torch.cuda.synchronize()
    want = torch.einsum("mhk,hnk->mhn", a[:, :, :K].double(), w.double())
    assert float((out.cpu().double() - want).abs().max()) < (1e-5 if dtype == "float32" else 5e-2)
