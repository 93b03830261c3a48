#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-MoE engine on ONE B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --design salepel [--sizes s,m]      another design beside Llama-MoE at equal sizes (see bench_design)
    python bench.py --design zufadra [--sizes s,m]      the Zufadra design beside a dense Llama at equal sizes
    python bench.py --design fugavik [--sizes s,m]      the Fugavik design beside Zufadra, Dumalix and Llama-MoE

The default run has the layer sizes of the LLaMA-MoE-3.5B (4/16) shape (32 layers, width 4096,
32/32 heads of 128, 16 experts top-4 of width 688, vocabulary 32000, context 4096) with random
bfloat16 weights, a batch of 8 and prompt lengths uniform in [128, 2048].  A "step" is one decode
step.  It prints ONE JSON line:

  value      decoded tokens a second: regions of exactly K steps each, timed on the device with CUDA
             events, repeated until at least a second has been timed; the median region counts
             (ms_per_step, with the fastest and slowest region under "spread"); the sampled tokens
             stay on the device between steps
  e2e        the same through transformer_b200.generate (as many steps as all regions together): host
             token lists in and out, the step's index arrays copied from pinned memory and the
             sampled tokens read back at every step
  prefill    one sequence of 2,048 tokens; frac = flops / time / the measured bf16 peak
  roofline   bytes the decode step has to read (every weight it uses once, the cache of the live
             requests) / its time, against the measured copy bandwidth
  points     decode tokens a second at batch 1 (a prompt of 1,088 tokens, the mean of the range) and
             64, each with its mean context, distinct experts per layer, fraction of the copy
             bandwidth and end-to-end figure

Every timed step reads far more than the 126 MB of L2 (all weights), so no L2 flush is needed.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = {   # BASELINE.json configs[2]
    "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 128, "intermediate_size": 688, "num_local_experts": 16,
    "num_experts_per_tok": 4, "max_position_embeddings": 4096, "vocab_size": 32000, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "tie_word_embeddings": False,
}
FULL_LAYERS = 32
PROMPT_MIN, PROMPT_MAX = 128, 2048
PREFILL_TOKENS = 2048
# The other shapes BASELINE.json names (configs[3], configs[4]); not the default and not the headline: further sizes
# for the same kernels.  name -> (config, layers of the full model, prompt length range)
OTHER_SHAPES = {
    "mixtral-8x7b": ({
        "model_type": "llama", "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "num_local_experts": 8,
        "num_experts_per_tok": 2, "max_position_embeddings": 32768, "vocab_size": 32000, "rms_norm_eps": 1e-5,
        "rope_theta": 1e6, "tie_word_embeddings": False}, 32, (512, 8192)),
    "mixtral-8x22b": ({
        "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 6144, "num_attention_heads": 48,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 16384, "num_local_experts": 8,
        "num_experts_per_tok": 2, "max_position_embeddings": 65536, "vocab_size": 32768, "rms_norm_eps": 1e-5,
        "rope_theta": 1e6, "tie_word_embeddings": False}, 56, (1, 16384)),
}
MIN_TIMED_SECONDS = 1.0     # the K-step region is repeated until this much has been timed
MAX_REGIONS = 40


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Clocks:
    """nvidia-smi sampling in the background while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid=None):
        """uuid: of the device the process runs on (cuda:0 of this process is rarely index 0 of a shared box)."""
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.gpu = f"GPU-{uuid}" if uuid else "0"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()     # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.file.close()
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def prefill_flops(c, T):
    L, d, nh, nkvh, dh = c["num_hidden_layers"], c["hidden_size"], c["num_attention_heads"], \
        c["num_key_value_heads"], c["head_dim"]
    E, k, di, V = c["num_local_experts"], c["num_experts_per_tok"], c["intermediate_size"], c["vocab_size"]
    per_layer = 2 * T * d * (nh + 2 * nkvh) * dh + 2 * T * nh * dh * d + 2 * T * d * E + 2 * T * k * 3 * d * di \
        + 4 * nh * dh * T * (T + 1) // 2
    return L * per_layer + 2 * d * V


def decode_bytes(c, distinct_experts_per_layer, context_tokens, elem=2):
    """Bytes one decode step must read: every weight it uses once + the cache of the live requests."""
    L, d, nh, nkvh, dh = c["num_hidden_layers"], c["hidden_size"], c["num_attention_heads"], \
        c["num_key_value_heads"], c["head_dim"]
    E, di, V = c["num_local_experts"], c["intermediate_size"], c["vocab_size"]
    fixed = L * (d * (nh + 2 * nkvh) * dh + nh * dh * d + E * d) * elem + L * 2 * d * 4 + d * 4 + V * d * elem
    experts = sum(distinct_experts_per_layer) * 3 * d * di * elem
    cache = L * context_tokens * 2 * nkvh * dh * elem
    return fixed + experts + cache


# ---- another design beside the closest existing model, at equal sizes (--design) ---------------------------------
def design_shapes(size):
    """(Salepel config, Llama-MoE config of equal width, depth, experts and attention output) for a named size."""
    d, L, H, dim, rot, vdim, rank, q_rank, window, mh, mdim, mvdim, E, ident, top, ff = {
        "s": (1024, 8, 8, 64, 32, 64, 256, 384, 1024, 4, 128, 256, 8, 1, 2, 512),
        "m": (2048, 8, 16, 128, 64, 128, 512, 768, 2048, 8, 128, 256, 16, 2, 4, 704),
    }[size]
    att = {"heads": H, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
           "mask": {"size": window}, "rot": {"base": 10000.0, "dims": rot}, "scale": (dim + rot) ** -0.5}
    mem = {"heads": mh, "dim": mdim, "vdim": mvdim, "gate_cap": 15.0}
    mlp = {"kind": "moe", "router": {"experts": E, "identity": ident, "top": top}, "expert": {"ff": ff, "limit": 7.0}}
    layers = []
    for i in range(L):      # of four layers: a latent of its own, the matrix memory, two that read the first one's latent
        if i % 4 == 1:
            layers.append({"type": "mlstm", "mixer": mem, "mlp": mlp})
        elif i % 4 == 0:
            layers.append({"type": "latent_attention", "mixer": att, "mlp": mlp})
        else:
            layers.append({"type": "latent_attention", "mixer": dict(att, kv_from=i - i % 4), "mlp": mlp})
    salepel = {"architecture": "Salepel", "vocab": 32000, "width": d, "norm": {"eps": 1e-6},
               "embedding": {"scale": 1.0}, "max_context": 8192, "layers": layers}
    llama = {"model_type": "llama", "num_hidden_layers": L, "hidden_size": d, "num_attention_heads": H * vdim // 128,
             "num_key_value_heads": max(1, H * vdim // 128 // 4), "head_dim": 128, "intermediate_size": ff,
             "num_local_experts": E, "num_experts_per_tok": top, "max_position_embeddings": 8192, "vocab_size": 32000,
             "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False}
    return salepel, llama


def zufadra_shapes(size):
    """(Zufadra config, dense Llama config of equal width, depth, heads and feed-forward) for a named size.  Layers
    alternate between the delta rule and the windowed attention, each followed by the dense feed-forward."""
    d, L, H, G, dim, window, rank, ff = {
        "s": (1024, 8, 8, 2, 128, 1024, 64, 2816),
        "m": (2048, 8, 16, 4, 128, 2048, 128, 5632),
    }[size]
    att = {"heads": H, "kv_heads": G, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 30.0,
           "mask": {"size": window, "keep_first": 4},
           "rot": {"base": 500000.0, "dims": dim // 2,
                   "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    mem = {"heads": H, "kv_heads": H, "dim": dim, "vdim": dim, "conv": 4, "decay_rank": rank, "gate_rank": rank}
    mlp = {"kind": "dense", "ff": ff}
    layers = [{"type": "channel_delta" if i % 2 == 0 else "attention", "mixer": mem if i % 2 == 0 else att, "mlp": mlp}
              for i in range(L)]
    zufadra = {"architecture": "Zufadra", "vocab": 32000, "width": d, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
               "logit_scale": 0.5, "embedding": {"scale": 8.0, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 7}},
               "max_context": 8192, "layers": layers}
    llama = {"model_type": "llama", "num_hidden_layers": L, "hidden_size": d, "num_attention_heads": H,
             "num_key_value_heads": G, "head_dim": dim, "intermediate_size": ff, "max_position_embeddings": 8192,
             "vocab_size": 32000, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False}
    return zufadra, llama


def dumalix_shapes(size):
    """(Dumalix config, Zufadra config of windowed attention alone, Salepel config) for a named size.  The Dumalix
    layers alternate between the latent attention and the chunked attention, each beside the clamped dense
    feed-forward; one pass over a repeated group of two layers.  The Zufadra model has the same width, depth, heads,
    head sizes and feed-forward, every layer a windowed attention (window = the chunk): the closest model for the
    attention kernels, the products and the feed-forward.  The Salepel model of the same size names has latents and
    heads of the same sizes: the closest model for the latent attention's kernels."""
    d, L, H, G, dim, chunk, lat_dim, rot, rank, ff = {
        "s": (1024, 8, 8, 2, 128, 1024, 64, 32, 256, 2816),
        "m": (2048, 8, 16, 4, 128, 2048, 128, 64, 512, 5632),
    }[size]
    att = {"heads": H, "kv_heads": G, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "conv": 4, "mask": {"size": chunk},
           "rot": {"base": 500000.0, "dims": dim // 2,
                   "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    lat = {"heads": H, "dim": lat_dim, "rot_dim": rot, "vdim": lat_dim, "kv_rank": rank, "scale": (lat_dim + rot) ** -0.5,
           "rot": {"base": 10000.0, "dims": rot, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    layers = [{"type": "latent_attention" if i % 2 == 0 else "attention", "mixer": lat if i % 2 == 0 else att, "mlp": mlp}
              for i in range(L)]
    dumalix = {"architecture": "Dumalix", "vocab": 32000, "width": d, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
               "loop": {"start": 2, "stop": 4, "times": 1}, "max_context": 8192, "layers": layers}
    zatt = {"heads": H, "kv_heads": G, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 30.0,
            "mask": {"size": chunk, "keep_first": 4},
            "rot": {"base": 500000.0, "dims": dim // 2,
                    "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    zufadra = {"architecture": "Zufadra", "vocab": 32000, "width": d, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
               "logit_scale": 0.5, "embedding": {"scale": 8.0, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 7}},
               "max_context": 8192,
               "layers": [{"type": "attention", "mixer": zatt, "mlp": {"kind": "dense", "ff": ff}} for _ in range(L)]}
    return dumalix, zufadra, design_shapes(size)[0]


def fugavik_shapes(size):
    """(Fugavik config, Zufadra config, Dumalix config, Llama-MoE config) for a named size.  The Fugavik layers go
    delta rule, attention, attention, latent attention, twice; the feed-forwards alternate between the dense pair and
    the experts.  Zufadra (delta rule, attention over the paged cache with a gate or a sink in the same kernels, blocks
    that norm what their parts produce, dense feed-forward) is the closest model for the delta rule, the attention, the
    norms and the dense products; Dumalix has the latent attention of the same kind (queries from one projection, plain
    causal); Llama-MoE the experts of the same sizes."""
    d, L, H, G, dim, lat_dim, rank, ff, E, top, eff = {
        "s": (1024, 8, 8, 2, 128, 64, 256, 2816, 8, 2, 512),
        "m": (2048, 8, 16, 4, 128, 128, 512, 5632, 16, 4, 704),
    }[size]
    att = {"heads": H, "kv_heads": G, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "v_mix": True,
           "rot": {"base": 500000.0, "dims": dim, "scaling": {"factor": 4.0}}}
    lat = {"heads": H, "dim": lat_dim, "vdim": lat_dim, "kv_rank": rank, "scale": lat_dim ** -0.5}
    mem = {"heads": H, "kv_heads": H, "dim": dim, "vdim": dim, "conv": 4}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}}
    kinds = [("delta", mem), ("attention", att), ("attention", att), ("latent_attention", lat)]
    layers = [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": dense if i % 2 == 0 else moe} for i in range(L)]
    fugavik = {"architecture": "Fugavik", "vocab": 32000, "width": d, "norm": {"eps": 1e-6}, "max_context": 8192,
               "layers": layers}
    return fugavik, zufadra_shapes(size)[0], dumalix_shapes(size)[0], design_shapes(size)[1]


def bench_design(args):
    """Prefill and decode throughput of another design beside the closest existing model of equal sizes, and the
    device time of every kernel family in one eager step of each (CUDA events around each launch).  One JSON line."""
    import torch
    import transformer_b200 as tb
    from transformer_b200.csrc import lib
    from transformer_b200.sampling import Sampler

    pk = peaks()
    T, B, ctx0, K, W = args.prefill_tokens, args.batch, 1024, args.steps, max(3, args.warmup)
    gen = torch.Generator().manual_seed(7)
    names, shapes = {"salepel": (("salepel", "llama_moe"), design_shapes),
                     "zufadra": (("zufadra", "llama_dense"), zufadra_shapes),
                     "dumalix": (("dumalix", "zufadra_attention", "salepel"), dumalix_shapes),
                     "fugavik": (("fugavik", "zufadra", "dumalix", "llama_moe"), fugavik_shapes)}[args.design]
    out = {"metric": f"prefill and decode tok/s, {names[0]} beside {' and '.join(names[1:])} at equal sizes", "unit": "tokens/s",
           "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic: random weights, random token ids",
           "peaks": pk, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx0, "steps": K, "warmup": W,
           "sizes": {}}
    for size in args.sizes.split(","):
        row = {}
        for name, cfg in zip(names, shapes(size)):
            room = max(T, B * (ctx0 + K * 8 + W + 80)) + 4096
            engine = tb.random_model(cfg, seed=0, dtype=args.dtype, max_tokens=room, max_slots=B + 2,
                                     max_step_tokens=max(8192, T))
            V = engine.spec.vocab
            sampler, greedy = Sampler(engine.device), tb.SampleArgs()
            ptoks = torch.randint(0, V, (T,), generator=gen).tolist()
            times = []
            for i in range(W + 5):
                s = engine.open()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                engine.step([s], [ptoks])
                e1.record()
                torch.cuda.synchronize()
                engine.close(s)
                if i >= W:
                    times.append(e0.elapsed_time(e1))
            p_ms = statistics.median(times)
            engine.use_tapes = False
            s = engine.open()
            with lib.timing() as tp:
                engine.step([s], [ptoks])
            engine.close(s)
            engine.use_tapes = True
            # decode: B sequences of ctx0 tokens, one token each per step, sampled tokens stay on the device
            slots = [engine.open() for _ in range(B)]
            logits = engine.step(slots, [torch.randint(0, V, (ctx0,), generator=gen).tolist() for _ in range(B)])
            ids = sampler.sample(logits, greedy)[0].clone()
            shape = [[0]] * B

            def one():
                lg = engine.step(slots, shape, device_tokens=ids)
                ids.copy_(sampler.sample(lg, greedy)[0])

            engine.use_graphs, engine.use_tapes = False, False
            one()
            with lib.timing() as td:
                one()
            engine.use_graphs, engine.use_tapes = True, True
            for _ in range(W):
                one()
            regions = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(K):
                    one()
                e1.record()
                torch.cuda.synchronize()
                regions.append(e0.elapsed_time(e1) / K)
            d_ms = statistics.median(regions)
            for sl in slots:
                engine.close(sl)
            weights = sum(t.numel() * t.element_size() for t in
                          {id(t): t for p in [engine.embed, engine.head_part, engine.final_norm] +
                           [q for l in engine.layers for q in l.parts().values()] for t in p.weights.values()}.values())
            row[name] = {
                "prefill_ms": p_ms, "prefill_tok_s": T / (p_ms * 1e-3), "decode_ms_per_step": d_ms,
                "decode_tok_s": B / (d_ms * 1e-3), "weight_bytes": weights, "cache_bytes": engine.cache.nbytes,
                "prefill_kernels_ms": {k: round(v, 4) for k, v in sorted(tp.ms.items(), key=lambda kv: -kv[1])},
                "prefill_kernel_calls": tp.calls,
                "decode_kernels_ms": {k: round(v, 4) for k, v in sorted(td.ms.items(), key=lambda kv: -kv[1])},
                "decode_kernel_calls": td.calls,
            }
            del engine
            torch.cuda.empty_cache()
        out["sizes"][size] = row
    print(json.dumps(out))
    return 0


def main():
    global PROMPT_MIN, PROMPT_MAX, PREFILL_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers of the same sizes (named in config)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points")
    ap.add_argument("--shape", default="llama-moe-3.5b", choices=["llama-moe-3.5b", *OTHER_SHAPES],
                    help="layer sizes: the benchmark's (default) or another shape BASELINE.json names")
    ap.add_argument("--prompt-max", type=int, default=0, help="longest prompt drawn (default: the shape's own)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    ap.add_argument("--design", default=None, choices=["salepel", "zufadra", "dumalix", "fugavik"],
                    help="instead of the default workload: this design beside the closest existing model at equal "
                         "sizes (prefill of --prefill-tokens, decode at --batch; sizes from --sizes)")
    ap.add_argument("--sizes", default="s,m", help="with --design: which of the named sizes (s, m)")
    args = ap.parse_args()
    if args.design is not None and args.impl == "ours":
        if args.gpus != 1:
            print(f"bench.py measures one GPU only (asked for {args.gpus})")
            return 2
        return bench_design(args)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "YdrMaster/transformer is a Rust workspace with git dependencies: no Rust toolchain, no "
                          "network and no Python package to install here (pip finds no setup.py or pyproject.toml)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library does no work on several GPUs (asked for {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import transformer_b200 as tb
    from transformer_b200.csrc import lib
    from transformer_b200.sampling import Sampler

    pk = peaks()
    shape, full_layers = SHAPE, FULL_LAYERS
    if args.shape != "llama-moe-3.5b":
        shape, full_layers, (PROMPT_MIN, PROMPT_MAX) = OTHER_SHAPES[args.shape]
        if args.layers == FULL_LAYERS:
            args.layers = shape["num_hidden_layers"]
    if args.prompt_max:
        PROMPT_MAX = max(PROMPT_MIN, args.prompt_max)
    PREFILL_TOKENS = args.prefill_tokens
    cfg = dict(shape, num_hidden_layers=args.layers)
    K, W, B = args.steps, args.warmup, args.batch
    gen = torch.Generator().manual_seed(1234)

    def lengths(n):
        return torch.randint(PROMPT_MIN, PROMPT_MAX + 1, (n,), generator=gen).tolist()

    def prompts_of(lens):
        return [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lens]

    batches = {B: lengths(B)}
    if not args.skip_points:
        batches.setdefault(1, [(PROMPT_MIN + PROMPT_MAX) // 2])     # one sequence: the mean of the range, not a draw
        batches.setdefault(64, lengths(64))
    # steps a run may take: warm-up and the regions (a second of them: some 500 steps of one sequence, 100 of 64)
    def most_steps(b):
        budget = max(K, 640 if b <= 16 else 160)
        return min(W + 2 + min(MAX_REGIONS * K, budget), cfg["max_position_embeddings"] - PROMPT_MAX - 8)
    room = max(sum((n + most_steps(len(ls)) + 8 + 63) // 64 * 64 for n in ls) for ls in batches.values())
    room = max(room, (PREFILL_TOKENS + 63) // 64 * 64)
    engine = tb.random_model(cfg, seed=0, dtype=args.dtype, max_tokens=room, max_slots=max(batches) + 1)
    sampler = Sampler(engine.device)
    greedy = tb.SampleArgs()
    dev = engine.device

    # ---- prefill of 2,048 tokens ---------------------------------------------------------------
    ptoks = prompts_of([PREFILL_TOKENS])[0]
    times = []
    for i in range(3 + 5):
        s = engine.open()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([s], [ptoks])
        e1.record()
        torch.cuda.synchronize()
        engine.close(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    p_ms = statistics.median(times)
    p_flops = prefill_flops(cfg, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (p_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": p_ms,
               "frac": p_flops / (p_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode ----------------------------------------------------------------------------------
    def decode_run(lens, with_clocks):
        b = len(lens)
        prompts = prompts_of(lens)
        slots = [engine.open() for _ in range(b)]
        logits = engine.step(slots, prompts)
        ids, _ = sampler.sample(logits, greedy)
        ids = ids.clone()
        shape = [[0]] * b

        def one():
            lg = engine.step(slots, shape, device_tokens=ids)
            nxt, _ = sampler.sample(lg, greedy)
            ids.copy_(nxt)

        # which experts does a step use?  (one eager step with the recorder, outside the timing)
        chosen = []
        engine.recorder = lambda name, run, t: chosen.append(t) if name == "moe.topk_idx" else None
        engine.use_graphs = False
        one()
        engine.use_graphs = True
        engine.recorder = None
        distinct = [int(torch.unique(t).numel()) for t in chosen]
        for _ in range(W):
            one()
        torch.cuda.synchronize()
        uuid = getattr(torch.cuda.get_device_properties(dev), "uuid", None)
        clk = Clocks(uuid)
        if with_clocks:
            clk.start()
            time.sleep(0.3)
        n0 = lib.launch_count
        regions, ctx_sum, steps_left = [], 0, most_steps(b) - W - 2
        while (sum(regions) < MIN_TIMED_SECONDS * 1e3 or not regions) and len(regions) < MAX_REGIONS and steps_left >= K:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before = sum(engine.cache.length(s) for s in slots)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(K):
                one()
            e1.record()
            torch.cuda.synchronize()
            regions.append(e0.elapsed_time(e1))
            ctx_sum += before + b * (K // 2)          # the region's mean context
            steps_left -= K
        launches = (lib.launch_count - n0) // len(regions)
        clocks = clk.stop() if with_clocks else None
        ms = statistics.median(regions)
        ctx_tokens = ctx_sum / len(regions)
        for s in slots:
            engine.close(s)
        # end to end through the public entry point: the same prompts, and as many decode steps as the device-timed
        # regions had in all (K of them would be a tenth of a second, mostly the clocks' recovery from the prompts)
        res = tb.generate(engine, prompts, max_steps=W + 1, stop_tokens=())        # warm-up
        res = tb.generate(engine, prompts, max_steps=K * len(regions) + 1, stop_tokens=())
        return {"tok_s": b * K / (ms * 1e-3), "ms_per_step": ms / K, "launches": launches, "clocks": clocks,
                "bytes": decode_bytes(cfg, distinct, ctx_tokens, 2 if args.dtype == "bfloat16" else 4),
                "distinct": sum(distinct) / max(1, len(distinct)), "ctx": ctx_tokens / b,
                "spread": [min(regions) / K, max(regions) / K], "regions": len(regions),
                "e2e": res.timing.decode_tokens / res.timing.decode_seconds,
                "h2d": int(getattr(engine, "last_h2d_bytes", 0))}

    main_run = decode_run(batches[B], True)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = main_run if b == B else decode_run(batches[b], False)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_hbm_frac"] = r["bytes"] / (r["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"]
            points[f"decode_b{b}_ms"] = r["ms_per_step"]
            points[f"decode_b{b}_mean_context"] = round(r["ctx"], 1)
            points[f"decode_b{b}_distinct_experts"] = round(r["distinct"], 2)
            points[f"decode_b{b}_e2e"] = r["e2e"]
    e2e_tok_s, h2d = main_run["e2e"], main_run["h2d"]

    achieved = main_run["bytes"] / (main_run["ms_per_step"] * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {B} ({'LLaMA-MoE-3.5B' if args.shape == 'llama-moe-3.5b' else args.shape} shape)",
        "value": main_run["tok_s"], "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": main_run["ms_per_step"], "higher_is_better": True,
        "spread": {"regions_of_k_steps": main_run["regions"], "ms_per_step_fastest": main_run["spread"][0],
                   "ms_per_step_slowest": main_run["spread"][1]},
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights ~N(0, 0.02) (counter-based, filled on the device), uniform-random token ids", "impl": "ours",
        "config": {
            "model": args.shape + "-shape", "layers": args.layers, "layers_full": full_layers,
            "width": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "experts": cfg["num_local_experts"],
            "experts_per_tok": cfg["num_experts_per_tok"], "expert_ffn": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "context": cfg["max_position_embeddings"], "global_batch": B, "prompt_len_min": PROMPT_MIN,
            "prompt_len_max": PROMPT_MAX, "mean_context": round(main_run["ctx"], 1), "seq_len": 1,
            "parallelism": "none", "l2": "every step reads all weights, far more than L2",
        },
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B + 4},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"],
                     "distinct_experts_per_layer": round(main_run["distinct"], 2)},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
