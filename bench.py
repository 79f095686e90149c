"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

The default run has the layer sizes of Llama-3.2-1B with random bfloat16 weights, 8 sequences
prefilled to 2,048 tokens each and then decoded (pool sized for a context of 4,096).  A step
is one decode step.  After W warm-up steps, blocks of exactly K steps are timed (up to five, as
many as the context leaves room for) and the median block is reported.  One JSON line is printed:

  value        decoded tokens a second, device-timed over exactly K steps (CUDA events)
  e2e          the same through LLMEngine.step(): host token ids in (pinned, copied every step),
               sampled token ids out (read back every step)
  prefill      one 2,048-token prompt in one step: tokens a second, ms, fraction of the bf16 peak
  roofline     bytes the decode step must read (every weight once + the live cache) / its time
  points       decode at batch 1 and 64: tokens a second, ms, bytes a step, fraction of the HBM peak
  more         other shapes and contexts (decode at 16 K and 32 K tokens; Llama-3.2-3B sizes: a prompt
               of 8,000 tokens, decode behind it, 64 sequences at 2 K); left out with --skip-more
  clocks       SM clock and throttle reasons sampled while the timed steps ran

Each timed step reads all weights (2.5 GB), far more than the 126 MB L2, so no flush is needed.
For --gpus > 1 it prints one line saying so and exits with 2.

``--impl reference`` times the reference's own engine (its unmodified package, looked for under
baseline/_ref, through its LLMEngine.for_model / add_request / step) on the same shape, batch, steps
and warm-up and prints the same line with "impl": "reference"; nothing of this package is imported
on that path.  Where the package is not there, or does not run, it prints why in one line.
"""

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = ROOT / "distributed-llm-inference_b200" / "config" / "shapes"
LLAMA_3_2_1B = json.loads((SHAPES / "llama-3.2-1b.json").read_text())
LLAMA_3_2_3B = json.loads((SHAPES / "llama-3.2-3b.json").read_text())
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE = 16
BLOCKS = 5  # timed blocks of --steps steps each; the median block is reported
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """nvidia-smi in the background while timed steps run; settings are only read."""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu: str = "0"):
        self.proc = None
        self.lines = []
        self.gpu = gpu  # what nvidia-smi -i takes: an index, or the UUID of the device this process computes on

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        self.lines += [line for line in out.splitlines() if line.strip()]
        self.proc = None

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0])), mx.append(float(f[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def device_id_for_smi() -> str:
    """The UUID of torch's device 0 (CUDA_VISIBLE_DEVICES may map it to any physical GPU of a shared
    machine; nvidia-smi counts physical ones), or "0" where torch does not tell."""
    import torch

    try:
        return "GPU-" + str(torch.cuda.get_device_properties(0).uuid)
    except Exception:
        return "0"


def weight_bytes(model):
    """Bytes of every tensor a decode step reads once (the embedding matrix counts once: it is
    the head; the few embedding rows gathered are negligible)."""
    seen, total = set(), 0
    for part in model.parts():
        for t in vars(part).values():
            if hasattr(t, "data_ptr") and hasattr(t, "numel") and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
    return total


def cache_bytes_per_token(model):
    from dli_b200.cache.needs import paged_need_of

    paged = [paged_need_of(n) for n in model.cache_needs()]
    return sum(2 * n.num_kv_heads * n.head_dim * model.dtype.itemsize for n in paged if n is not None)


def prefill_flops(cfg, layers, tokens):
    H, I, d, nh, nkv, V = (cfg[k] for k in ("hidden_size", "intermediate_size", "head_dim", "num_attention_heads", "num_key_value_heads", "vocab_size"))
    per_token = 2 * (H * (nh + 2 * nkv) * d + nh * d * H + 3 * H * I)
    attention = 2 * tokens * tokens * d * nh  # QK^T and PV over the causal half
    return layers * (tokens * per_token + attention) + 2 * H * V


def timed_blocks(steps: int, warmup: int, room: int) -> int:
    """How many blocks of ``steps`` steps fit into ``room`` more tokens of context after the warm-up."""
    return max(1, min(BLOCKS, (room - warmup - 2) // max(1, steps)))


def make_engine(model, batch, prompt_len=PROMPT_LEN, context=CONTEXT):
    from dli_b200 import LLMEngine, SchedulerConfig

    pages = batch * (context // PAGE) + 8
    return LLMEngine.for_model(model, num_blocks=pages, block_size=PAGE, config=SchedulerConfig(max(batch, 1), min(prompt_len, 8192)),
                               enable_prefix_caching=False, watermark=0.0)


def decode_device_timed(model, batch, steps, warmup, sampler_clock=None, graphs=True, prompt_len=PROMPT_LEN, context=CONTEXT,
                        portion=2048, blocks=None, sampling=None):
    """Blocks of K decode steps timed on the device: step function plus sampling (greedy, or with ``sampling``:
    SamplingParams that every request gets, bound to its state slot as the engine binds them).  Each step runs
    on the ids the step before sampled, taken on the device; the host reads every step's ids, one
    step late (the engine's own way of stepping).  Prompts are prefilled in portions of ``portion``."""
    import torch

    from dli_b200.cache import UNKNOWN_TOKEN
    from dli_b200.engine import ModelRunner, StepEntry
    from dli_b200.kernels import ops
    from dli_b200.sampling import Sampler, SamplingParams

    runner = ModelRunner(model, num_pages=batch * (context // PAGE) + 8, page_size=PAGE, max_requests=batch,
                         enable_prefix_caching=False, watermark=0.0, cuda_graphs=graphs)
    sampler = Sampler(model.device, max_requests=batch if sampling else 0)
    g = torch.Generator().manual_seed(1)
    vocab = model.spec.vocab_size
    params = [SamplingParams()] * batch
    for b in range(batch if sampling else 0):
        sampler.bind(b, sampling, (sampling.seed or 0) + b, 0)

    def sample_rows(logits):
        if sampling:
            return sampler.sample_slots_async(logits, list(range(batch)), all_greedy=False)
        return sampler.sample_async(logits, params, [0] * batch, [0] * batch)

    tokens = []
    for b in range(batch):
        prompt = torch.randint(1000, vocab, (prompt_len,), generator=g).tolist()
        runner.manager.allocate(b, prompt)
        for at in range(0, prompt_len, portion):
            part = prompt[at : at + portion]
            logits = runner.step([StepEntry(b, part, [len(part) - 1] if at + portion >= prompt_len else [])])
        tokens.append(sampler.sample(logits, params[:1], [0], [0])[0])

    def launch(prev):
        """One decode step of every request, launched on the ids the step before left on the device
        (``prev``: PendingTokens), as LLMEngine.step does; the host reads those ids afterwards."""
        entries = []
        for b in range(batch):
            runner.manager.append_slots(b, [UNKNOWN_TOKEN])  # no prefix index in this run: the id is never needed
            entries.append(StepEntry(b, [0], [0], token_src=b))
        return sample_rows(runner.step(entries, borrow=True, token_source=prev.device_ids))

    # the first step runs on ids the host knows
    for b in range(batch):
        runner.manager.append_slots(b, [tokens[b]])
    flight = sample_rows(runner.step([StepEntry(b, [tokens[b]], [0]) for b in range(batch)], borrow=True))

    def one_step(flight):
        ahead = launch(flight)
        ids = flight.result()  # this step's tokens reach the host while the next step runs
        assert len(ids) == batch
        return ahead

    for _ in range(warmup):
        flight = one_step(flight)
    flight.result()
    torch.cuda.synchronize()
    if sampler_clock:
        sampler_clock.start()
    runs = []
    for _ in range(blocks or timed_blocks(steps, warmup, context - prompt_len)):
        ctx_start = runner.manager.num_tokens(0)
        launches = ops.launch_count
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            flight = one_step(flight)
        end.record()
        torch.cuda.synchronize()
        runs.append({"ms": start.elapsed_time(end) / steps, "launches": ops.launch_count - launches, "mean_ctx": ctx_start + steps / 2})
    flight.result()
    if sampler_clock:
        sampler_clock.stop()
    for b in range(batch):
        runner.manager.free(b)
    del runner
    torch.cuda.empty_cache()
    runs.sort(key=lambda r: r["ms"])
    mid = runs[len(runs) // 2]
    return {**mid, "tok_s": batch * 1000.0 / mid["ms"], "blocks": len(runs), "block_ms": [round(r["ms"], 4) for r in runs]}


def decode_end_to_end(model, batch, steps, warmup):
    """Blocks of K steps of LLMEngine.step(): every step copies its token ids and tables from pinned
    host memory to the device and reads the sampled ids back.  The median block is reported."""
    import torch

    from dli_b200 import SamplingParams

    eng = make_engine(model, batch)
    g = torch.Generator().manual_seed(2)
    for b in range(batch):
        eng.add_request(f"r{b}", torch.randint(1000, model.spec.vocab_size, (PROMPT_LEN,), generator=g).tolist(),
                        SamplingParams(max_tokens=CONTEXT - PROMPT_LEN, ignore_eos=True))
    while any(r.num_computed_tokens < PROMPT_LEN for r in eng.scheduler.running + list(eng.scheduler.waiting)):
        eng.step()
    for _ in range(warmup):
        eng.step()
    times = []
    for _ in range(timed_blocks(steps, warmup, CONTEXT - PROMPT_LEN)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            out = eng.step()
            assert len(out) == batch
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    h2d = eng.runner.uploader.bytes_last  # what the last step copied from pinned memory: token ids, positions, lengths, slots, block tables
    while eng.has_unfinished():
        for rid in [r.request_id for r in eng.scheduler.running]:
            eng.abort(rid)
    return {"value": batch * steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch, "ms_per_step": dt / steps * 1e3}


def prefill_timed(model, cfg, layers, peak_tflops, reps=5, warmup=3, tokens=PROMPT_LEN, graphs=True):
    import torch

    from dli_b200.engine import ModelRunner, StepEntry

    runner = ModelRunner(model, num_pages=tokens // PAGE + 8, page_size=PAGE, max_requests=2, enable_prefix_caching=False, watermark=0.0,
                         cuda_graphs=graphs)
    g = torch.Generator().manual_seed(3)
    times = []
    for i in range(warmup + reps):
        prompt = torch.randint(1000, model.spec.vocab_size, (tokens,), generator=g).tolist()
        runner.manager.allocate("p", prompt)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("p", prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        runner.manager.free("p")
    del runner
    torch.cuda.empty_cache()
    ms = statistics.median(times)
    flops = prefill_flops(cfg, layers, tokens)
    return {"value": tokens * 1000.0 / ms, "tokens": tokens, "ms": ms, "frac": flops / (ms * 1e-3) / (peak_tflops * 1e12),
            "flops": flops, "unit": "tokens/s"}


def sampling_timed(vocab, reps=5, per_graph=8):
    """Microseconds of the sampling kernel alone, by what the rows ask for, at 1, 8 and 64 rows of ``vocab`` logits:
    a graph of ``per_graph`` launches, replayed ``reps`` times between two events."""
    import torch

    from dli_b200.kernels import ops

    dev = "cuda:0"
    modes = {"greedy": None, "temperature": (0.8, -1, 1.0), "top_k_50": (0.8, 50, 1.0), "top_p_0.9": (0.8, -1, 0.9), "top_k_50_top_p_0.9": (0.8, 50, 0.9)}
    out = {}
    for rows in (1, 8, 64):
        g = torch.Generator().manual_seed(rows)
        logits = (torch.randn(rows, vocab, generator=g) * 3).to(dev)
        ids = torch.empty(rows, dtype=torch.int32, device=dev)
        seed, draw = torch.arange(rows, dtype=torch.int64, device=dev), torch.zeros(rows, dtype=torch.int64, device=dev)
        for name, mode in modes.items():
            if mode is None:
                fn = lambda: ops.sample(ids, logits)
            else:
                t, k, p = (torch.full((rows,), mode[0], device=dev), torch.full((rows,), mode[1], dtype=torch.int32, device=dev),
                           torch.full((rows,), mode[2], device=dev))
                fn = lambda t=t, k=k, p=p: ops.sample(ids, logits, t, k, p, seed, draw)
            fn()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(per_graph):
                    fn()
            graph.replay()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(reps):
                graph.replay()
            end.record()
            torch.cuda.synchronize()
            out[f"rows{rows}_{name}"] = round(start.elapsed_time(end) * 1000.0 / reps / per_graph, 1)
    return out


def decode_point(model, batch, steps, warmup, hbm_gbs, **kw):
    """A decode measurement as a record: tokens a second, ms a step, the bytes a step has to read
    (every weight once and the live cache at the block's mean context) and their share of the HBM peak."""
    run = decode_device_timed(model, batch, steps, warmup, **kw)
    step_bytes = weight_bytes(model) + batch * run["mean_ctx"] * cache_bytes_per_token(model)
    gbs = step_bytes / (run["ms"] * 1e-3) / 1e9
    return {"tok_s": round(run["tok_s"], 1), "ms": round(run["ms"], 4), "bytes_per_step": int(step_bytes), "gb_s": round(gbs, 1),
            "frac": round(gbs / hbm_gbs, 4), "mean_ctx": run["mean_ctx"]}


def more_points(model_1b, steps, warmup, pk):
    """Beyond the headline: longer contexts at the 1B sizes, and the Llama-3.2-3B sizes (a prompt of 8,000
    tokens in one step, decode behind it, 64 sequences at a context of 2 K)."""
    import torch

    import dli_b200

    from dli_b200.sampling import SamplingParams

    steps = min(steps, 32)
    out = {}
    # the headline step with every request sampling at temperature 0.8 among the 50 likeliest tokens and 0.9 of their mass
    out["decode_b8_sampled"] = decode_point(model_1b, 8, steps, warmup, pk["hbm_gbs"], blocks=1,
                                            sampling=SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1))
    # a short prompt in one step: launched kernel by kernel the host needs 2.3 ms for it; once the shape has come
    # often enough the step is replayed from a graph (engine/graphs.py, MixedGraph)
    short = prefill_timed(model_1b, LLAMA_3_2_1B, LLAMA_3_2_1B["num_hidden_layers"], pk["bf16_tflops"], reps=5, warmup=40, tokens=256)
    out["prefill_256"] = {"tok_s": round(short["value"], 1), "ms": round(short["ms"], 4), "frac": round(short["frac"], 4)}
    for name, batch, ctx in (("decode_b8_ctx16k", 8, 16384), ("decode_b1_ctx32k", 1, 32768), ("decode_b8_ctx32k", 8, 32768)):
        out[name] = decode_point(model_1b, batch, steps, warmup, pk["hbm_gbs"], prompt_len=ctx, context=ctx + 512, blocks=1)
    cfg = LLAMA_3_2_3B
    model = dli_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    pre = prefill_timed(model, cfg, cfg["num_hidden_layers"], pk["bf16_tflops"], reps=3, warmup=2, tokens=8000)
    out["3b_prefill_8000"] = {"tok_s": round(pre["value"], 1), "ms": round(pre["ms"], 3), "tflops": round(pre["flops"] / pre["ms"] / 1e9, 1),
                              "frac": round(pre["frac"], 4)}
    out["3b_decode_b1_ctx8k"] = decode_point(model, 1, steps, warmup, pk["hbm_gbs"], prompt_len=8000, context=8192 + 512, blocks=1)
    out["3b_decode_b8_ctx8k"] = decode_point(model, 8, steps, warmup, pk["hbm_gbs"], prompt_len=8000, context=8192 + 512, blocks=1)
    out["3b_decode_b64_ctx2k"] = decode_point(model, 64, steps, warmup, pk["hbm_gbs"], prompt_len=2048, context=2048 + 512, blocks=1)
    return out


# ----------------------------------------------------------------------------- --design: another architecture beside Llama


def pazenex_sizes(width, heads, kv_heads, dim, ssm_heads, state, groups, ff, vocab=32000):
    """A Pazenex model of eight layer runs (attention, Mamba-2, attention, Mamba-2, the four run twice) and the Llama
    configuration of the same width, heads, feed-forward size and number of layers."""
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
           "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim**-0.5,
                     "rot": {"base": 500000.0, "dims": dim, "scaling": {"factor": 8.0}}}}
    ssm = {"type": "mamba2", "mlp": {"kind": "dense", "ff": ff},
           "mixer": {"heads": ssm_heads, "vdim": 64, "state": state, "groups": groups, "conv": 4, "norm_groups": groups}}
    pz = {"architecture": "Pazenex", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [att, ssm, att, ssm],
          "loop": {"start": 0, "stop": 4, "times": 2}}
    llama = dict(LLAMA_3_2_1B, hidden_size=width, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=dim,
                 intermediate_size=ff, num_hidden_layers=8, vocab_size=vocab, tie_word_embeddings=False)
    return pz, llama


DESIGN_SIZES = {
    "w1024": dict(width=1024, heads=16, kv_heads=4, dim=64, ssm_heads=32, state=64, groups=4, ff=4096),
    "w2048": dict(width=2048, heads=32, kv_heads=8, dim=64, ssm_heads=64, state=128, groups=8, ff=8192),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ssm_heads=128, state=128, groups=8, ff=14336),
}


def all_weight_bytes(model):
    seen, total = set(), 0

    def walk(v):
        nonlocal total
        if hasattr(v, "data_ptr") and hasattr(v, "numel"):
            if v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                total += v.numel() * v.element_size()
        elif isinstance(v, dict):
            for x in v.values():
                walk(x)

    for part in model.parts():
        for v in vars(part).values():
            walk(v)
    return total


def time_kernel(fn, reps=7, warmup=3):
    """Median device time of fn() in microseconds; a 256 MB buffer is written between calls, so nothing stays in L2."""
    import torch

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    times = []
    for i in range(warmup + reps):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end) * 1e3)
    return statistics.median(times)


def design_kernels(size, pk, tokens=4096, seqs=64):
    """Every kernel of the new parts beside the like kernel of the Llama parts, at one size: a prompt portion of ``tokens``
    tokens and a decode step of ``seqs`` sequences.  us, the bytes (or operations) the kernel has to move, and the share
    of the measured HBM peak (of the CUDA cores' float32 rate for the scan over a portion)."""
    import torch

    from dli_b200.kernels import ops

    dev, bf = "cuda", torch.bfloat16
    W, nh, nkv, d = size["width"], size["heads"], size["kv_heads"], size["dim"]
    Hs, P, N, G, taps, ff = size["ssm_heads"], 64, size["state"], size["groups"], 4, size["ff"]
    inner = Hs * P
    C = inner + 2 * G * N
    out = {}

    def record(name, us, nbytes, like=None, flops=None):
        rec = {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        if flops is not None:
            rec["tflops_fp32"] = round(flops / us / 1e6, 2)
            rec["simt_frac"] = round(flops / us / 1e6 / SIMT_FP32_TFLOPS, 3)
        if like:
            rec["like"] = like
        out[name] = rec

    for label, n, S in (("portion", tokens, 1), ("decode", seqs, seqs)):
        q_lens = [n // S] * S
        q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        seq_of = torch.repeat_interleave(torch.arange(S, dtype=torch.int32), n // S).to(dev)
        slot = torch.arange(S, dtype=torch.int32, device=dev)
        positions = torch.arange(n, dtype=torch.int32, device=dev) % (n // S) + (0 if S == 1 else 2047)
        h = torch.randn(n, W, device=dev)
        a = torch.randn(n, W, device=dev).to(bf)
        w1, w2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
        y = torch.empty(n, W, dtype=bf, device=dev)
        record(f"{label}.post_add_layernorm", time_kernel(lambda: ops.post_add_layernorm(y, h, a, w1, w2, 1e-6, 1e-6)), n * W * 12, "add_rmsnorm")
        record(f"{label}.add_rmsnorm", time_kernel(lambda: ops.add_rmsnorm(y, h, a, w1, 1e-6)), n * W * 12)
        # attention preparation
        page, pages = 16, (n if S == 1 else S) // 16 + 2
        slots = torch.arange(n, dtype=torch.int32, device=dev)
        kp, vp = (torch.zeros(pages + n // 16, nkv, page, d, dtype=bf, device=dev) for _ in range(2))
        inv = (1.0 / (500000.0 ** (torch.arange(0, d, 2).float() / d))).to(dev)
        proj = torch.randn(n, (2 * nh + nkv) * d, device=dev).to(bf)
        wq, wk = torch.ones(nh * d, device=dev), torch.ones(nkv * d, device=dev)
        moved = n * ((nh + nkv) * d * 2 + (nh + 2 * nkv) * d * 2)
        record(f"{label}.qk_norm_rotary_store", time_kernel(lambda: ops.qk_norm_rotary_store(proj, wq, wk, 1e-6, positions, inv, slots, kp, vp, nh, nkv, d, d, page)),
               moved, "rotary_store")
        qkv = torch.randn(n, (nh + 2 * nkv) * d, device=dev).to(bf)
        record(f"{label}.rotary_store", time_kernel(lambda: ops.rotary_store(qkv, positions, inv, slots, kp, vp, nh, nkv, d, d, page)),
               n * ((nh + nkv) * d * 4 + nkv * d * 4))
        att = torch.randn(n, nh * d, device=dev).to(bf)
        gate = proj[:, (nh + nkv) * d :]
        record(f"{label}.sigmoid_gate", time_kernel(lambda: ops.sigmoid_gate(att, gate)), n * nh * d * 6, "silu_mul")
        up = torch.randn(n, ff, device=dev).to(bf)
        record(f"{label}.activation_relu2", time_kernel(lambda: ops.activation(up, "relu2")), n * ff * 4, "silu_mul")
        gu = torch.randn(n, 2 * ff, device=dev).to(bf)
        act = torch.empty(n, ff, dtype=bf, device=dev)
        record(f"{label}.silu_mul", time_kernel(lambda: ops.silu_mul(act, gu)), n * ff * 6)
        # state-space mixer
        u = torch.randn(n, inner + C + Hs, device=dev).to(bf)
        xbc = torch.empty(n, C, dtype=bf, device=dev)
        cw, cb = torch.randn(taps, C, device=dev), torch.randn(C, device=dev)
        cstate = torch.zeros(S, taps - 1, C, dtype=bf, device=dev)
        record(f"{label}.causal_conv_silu", time_kernel(lambda: ops.causal_conv_silu(xbc, u, inner, cw, cb, cstate, seq_of, q_start, slot)),
               n * C * 4 + (S * (taps - 1) * C * 2 if S > 1 else 0), "silu_mul")
        state = torch.zeros(S, Hs, P, N, device=dev)
        ys = torch.empty(n, inner, device=dev)
        dtb, al, dk = torch.zeros(Hs, device=dev), torch.zeros(Hs, device=dev), torch.ones(Hs, device=dev)
        scan_us = time_kernel(lambda: ops.ssm_scan(ys, xbc, u, inner + C, dtb, al, dk, state, q_start, slot, G, max_len=n // S))
        scan_bytes = S * Hs * N * P * 8 + n * (C * 2 + inner * 4)
        record(f"{label}.ssm_scan", scan_us, scan_bytes, "decode attention" if S > 1 else "prefill attention", flops=5.0 * n * Hs * N * P)
        gated = torch.empty(n, inner, dtype=bf, device=dev)
        nw = torch.ones(inner, device=dev)
        record(f"{label}.gated_group_rmsnorm", time_kernel(lambda: ops.gated_group_rmsnorm(gated, ys, u, 0, nw, G, 1e-6)), n * inner * 8, "add_rmsnorm")
    return out


def sugonex_sizes(width, heads, dim, rot_dim, kv_rank, window, delta_heads, delta_kv_heads, delta_dim, ff, pz, vocab=32000):
    """A Sugonex model of eight layer runs (windowed latent attention, delta rule, latent attention with the rotated key
    part, delta rule; the four run twice) and the Pazenex configuration of the same width, heads, feed-forward size and
    number of layer runs (``pz``: its attention and state-space sizes)."""
    def mlp():
        return {"kind": "dense", "ff": ff}

    win = {"type": "latent_attention_2", "mlp": mlp(),
           "mixer": {"heads": heads, "dim": dim + rot_dim, "vdim": dim, "kv_rank": kv_rank + rot_dim, "scale": (dim + rot_dim) ** -0.5, "mask": {"size": window}}}
    rot = {"type": "latent_attention", "mlp": mlp(),
           "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": dim, "kv_rank": kv_rank, "scale": (dim + rot_dim) ** -0.5,
                     "rot": {"base": 500000.0, "dims": rot_dim}}}
    dl = {"type": "delta", "mlp": mlp(),
          "mixer": {"heads": delta_heads, "kv_heads": delta_kv_heads, "dim": delta_dim, "vdim": delta_dim, "conv": 4}}
    sg = {"architecture": "Sugonex", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [win, dl, rot, dl],
          "loop": {"start": 0, "stop": 4, "times": 2}, "logit_scale": 0.5, "logit_softcap": 30.0}
    pazenex, _ = pazenex_sizes(width=width, heads=heads, ff=ff, vocab=vocab, **pz)
    return sg, pazenex


# the cached row (kv_rank + rot_dim) is 128, 256 and 256 numbers: what this engine's tensor-core attention kernels take
SUGONEX_SIZES = {
    "w1024": dict(width=1024, heads=16, dim=64, rot_dim=32, kv_rank=96, window=1024, delta_heads=8, delta_kv_heads=4, delta_dim=128, ff=4096,
                  pz=dict(kv_heads=4, dim=64, ssm_heads=32, state=64, groups=4)),
    "w2048": dict(width=2048, heads=16, dim=128, rot_dim=64, kv_rank=192, window=1024, delta_heads=16, delta_kv_heads=8, delta_dim=128, ff=8192,
                  pz=dict(kv_heads=4, dim=128, ssm_heads=64, state=128, groups=8)),
    "w4096": dict(width=4096, heads=32, dim=128, rot_dim=64, kv_rank=192, window=1024, delta_heads=32, delta_kv_heads=16, delta_dim=128, ff=14336,
                  pz=dict(kv_heads=8, dim=128, ssm_heads=128, state=128, groups=8)),
}


def sugonex_kernels(size, pk, tokens=4096, seqs=64):
    """Every kernel of the Sugonex parts beside the like kernel of the Pazenex (or Llama) parts, at one size: a prompt
    portion of ``tokens`` tokens and a decode step of ``seqs`` sequences at a context of 2,048.  us, the bytes (or
    operations) the kernel has to move, and the share of the measured HBM peak (of the CUDA cores' float32 rate for the
    scans over a portion, of the measured bf16 rate for attention over a portion)."""
    import torch

    from dli_b200.cache.pools import LayerCache
    from dli_b200.engine.batch import GroupView, StepBatch
    from dli_b200.kernels import attention as attn
    from dli_b200.kernels import gemm, ops

    dev, bf = "cuda", torch.bfloat16
    W, nh, d, dr, r, ff = size["width"], size["heads"], size["dim"], size["rot_dim"], size["kv_rank"], size["ff"]
    Hd, Gd, dd = size["delta_heads"], size["delta_kv_heads"], size["delta_dim"]
    pz = size["pz"]
    row = r + dr
    out = {}

    def record(name, us, nbytes, like=None, flops=None, tensor=False):
        rec = {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        if flops is not None and tensor:
            rec["tflops_bf16"] = round(flops / us / 1e6, 1)
            rec["bf16_frac"] = round(flops / us / 1e6 / pk["bf16_tflops"], 3)
        elif flops is not None:
            rec["tflops_fp32"] = round(flops / us / 1e6, 2)
            rec["simt_frac"] = round(flops / us / 1e6 / SIMT_FP32_TFLOPS, 3)
        if like:
            rec["like"] = like
        out[name] = rec

    def attention_batch(S, q_len, context, page=16):
        """A batch of S sequences that each bring q_len tokens and end at ``context`` keys, in pages of their own."""
        n = S * q_len
        width = -(-context // page)
        tables = torch.arange(S * width, dtype=torch.int32, device=dev).view(S, width)
        q_start = torch.arange(S + 1, dtype=torch.int32, device=dev) * q_len
        kv_len = torch.full((S,), context, dtype=torch.int32, device=dev)
        seq_of = torch.repeat_interleave(torch.arange(S, dtype=torch.int32), q_len).to(dev)
        positions = (torch.arange(n, dtype=torch.int32) % q_len + (context - q_len)).to(dev)
        slots = (seq_of * width * page + positions).to(torch.int32)
        batch = StepBatch(n=n, num_seqs=S, num_single=S if q_len == 1 else 0, token_ids=positions, positions=positions, seq_of_token=seq_of,
                          q_start=q_start, kv_len=kv_len, state_slot=torch.arange(S, dtype=torch.int32, device=dev), logit_rows=positions[:0],
                          groups=[GroupView(tables, slots)], q_lens=[q_len] * S, starts=[context - q_len] * S, state_slots=list(range(S)),
                          max_q_len=q_len, max_kv_len=context, max_kv_len_single=context if q_len == 1 else 0)
        return batch, S * width

    for label, n, S in (("portion", tokens, 1), ("decode", seqs, seqs)):
        q_len = n // S
        context = tokens if S == 1 else 2048
        q_start = torch.arange(S + 1, dtype=torch.int32, device=dev) * q_len
        seq_of = torch.repeat_interleave(torch.arange(S, dtype=torch.int32), q_len).to(dev)
        slot = torch.arange(S, dtype=torch.int32, device=dev)
        # the norm in front of both branches, with both branches' outputs of the layer before
        h = torch.randn(n, W, device=dev)
        a, b = torch.randn(n, W, device=dev).to(bf), torch.randn(n, W, device=dev).to(bf)
        w1, w2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
        y1, y2 = torch.empty(n, W, dtype=bf, device=dev), torch.empty(n, W, dtype=bf, device=dev)
        record(f"{label}.add_rmsnorm_pair", time_kernel(lambda: ops.add_rmsnorm_pair(y1, y2, h, a, b, w1, w2, 1e-6)), n * W * 16, "post_add_layernorm")
        record(f"{label}.post_add_layernorm", time_kernel(lambda: ops.post_add_layernorm(y1, h, a, w1, w2, 1e-6, 1e-6)), n * W * 12)
        # attention over the latent: preparation, the heads' products, the attention kernels, the gate
        batch, pages = attention_batch(S, q_len, context)
        pool = torch.randn(pages + 1, 1, 16, row, device=dev).to(bf)
        cache = LayerCache(0, pool, pool, 16)
        proj = torch.randn(n, nh * (d + dr) + row + nh * d, device=dev).to(bf)
        q = torch.empty(n, nh * row, dtype=bf, device=dev)
        wn = torch.ones(r, device=dev)
        inv = (1.0 / (500000.0 ** (torch.arange(0, dr, 2).float() / dr))).to(dev)
        slots = batch.groups[0].slots
        record(f"{label}.latent_prep", time_kernel(lambda: ops.latent_prep(q, proj, wn, 1e-6, batch.positions, inv, slots, pool, nh, d, dr, r, dr, 16)),
               n * ((nh * dr + row) * 4), "qk_norm_rotary_store")
        wuk = (torch.randn(nh, d, r, device=dev) * 0.05).to(bf)
        record(f"{label}.heads_product_uk", time_kernel(lambda: gemm.heads_product(proj[:, : nh * (d + dr)].view(n, nh, d + dr)[:, :, :d], wuk,
                                                                                   q.view(n, nh, row)[:, :, :r])),
               n * nh * (d + r) * 2 + nh * d * r * 2, flops=2.0 * n * nh * d * r, tensor=True)
        lat = torch.empty(n, nh * row, dtype=bf, device=dev)
        causal = (context * (context + 1) / 2) if S == 1 else float(context)
        att_us = time_kernel(lambda: attn.paged_attention(lat, q, cache, batch, nh, row**-0.5, None))
        record(f"{label}.latent_attention", att_us, S * context * row * 2 + n * nh * row * 4, "sink attention", flops=4.0 * S * causal * nh * row, tensor=True)
        # its like: Pazenex's attention at equal heads (grouped-query, separate values)
        pd, pkv = pz["dim"], pz["kv_heads"]
        kp, vp = (torch.randn(pages + 1, pkv, 16, pd, device=dev).to(bf) for _ in range(2))
        pq, po = torch.randn(n, nh * pd, device=dev).to(bf), torch.empty(n, nh * pd, dtype=bf, device=dev)
        gqa_us = time_kernel(lambda: attn.paged_attention(po, pq, LayerCache(0, kp, vp, 16), batch, nh, pd**-0.5, None, sink=0.0))
        record(f"{label}.sink_attention", gqa_us, S * context * pkv * pd * 4 + n * nh * pd * 4, flops=4.0 * S * causal * nh * pd, tensor=True)
        wuv = (torch.randn(nh, r, d, device=dev) * 0.05).to(bf)
        o = torch.empty(n, nh * d, dtype=bf, device=dev)
        record(f"{label}.heads_product_uv", time_kernel(lambda: gemm.heads_product(lat.view(n, nh, row)[:, :, :r], wuv, o.view(n, nh, d))),
               n * nh * (d + r) * 2 + nh * d * r * 2, flops=2.0 * n * nh * d * r, tensor=True)
        gate = proj[:, nh * (d + dr) + row :]
        record(f"{label}.sigmoid_gate", time_kernel(lambda: ops.sigmoid_gate(o, gate)), n * nh * d * 6)
        # gated feed-forward's activation
        gu = torch.randn(n, 2 * ff, device=dev).to(bf)
        act = torch.empty(n, ff, dtype=bf, device=dev)
        record(f"{label}.gelu_mul", time_kernel(lambda: ops.silu_mul(act, gu, True, "gelu_tanh")), n * ff * 6, "silu_mul")
        record(f"{label}.silu_mul", time_kernel(lambda: ops.silu_mul(act, gu, True)), n * ff * 6)
        # delta rule: convolution, scan, norm with the gate behind it
        taps, qk, inner = 4, Gd * dd, Hd * dd
        C = 2 * qk + inner
        u = torch.randn(n, C + inner + 2 * Hd, device=dev).to(bf)
        qkv = torch.empty(n, C, dtype=bf, device=dev)
        cw = torch.randn(taps, C, device=dev)
        cstate = torch.zeros(S, taps - 1, C, dtype=bf, device=dev)
        record(f"{label}.causal_conv_silu", time_kernel(lambda: ops.causal_conv_silu(qkv, u, 0, cw, None, cstate, seq_of, q_start, slot)),
               n * C * 4 + (S * (taps - 1) * C * 2 if S > 1 else 0))
        state = torch.zeros(S, Hd, dd, dd, device=dev)
        os_ = torch.empty(n, inner, device=dev)
        dtb, al = torch.zeros(Hd, device=dev), torch.full((Hd,), -3.0, device=dev)
        scan_us = time_kernel(lambda: ops.delta_rule_scan(os_, qkv, u, C + inner, C + inner + Hd, dtb, al, state, seq_of, q_start, slot, Gd, dd, 1e-6, max_len=q_len))
        record(f"{label}.delta_rule_scan", scan_us, S * Hd * dd * dd * 8 + n * (C * 2 + inner * 4), "ssm_scan", flops=8.0 * n * Hd * dd * dd)
        # its like: the state-space scan of the Pazenex model of this size
        Hs, P, N, G = pz["ssm_heads"], 64, pz["state"], pz["groups"]
        sin, sC = Hs * P, Hs * P + 2 * G * N
        su = torch.randn(n, sin + sC + Hs, device=dev).to(bf)
        xbc = torch.randn(n, sC, device=dev).to(bf)
        sstate = torch.zeros(S, Hs, P, N, device=dev)
        ys = torch.empty(n, sin, device=dev)
        z3 = torch.zeros(Hs, device=dev)
        ssm_us = time_kernel(lambda: ops.ssm_scan(ys, xbc, su, sin + sC, z3, z3, z3 + 1, sstate, q_start, slot, G, max_len=q_len))
        record(f"{label}.ssm_scan", ssm_us, S * Hs * N * P * 8 + n * (sC * 2 + sin * 4), flops=5.0 * n * Hs * N * P)
        gated = torch.empty(n, inner, dtype=bf, device=dev)
        nw = torch.ones(inner, device=dev)
        record(f"{label}.group_norm_gate_after", time_kernel(lambda: ops.gated_group_rmsnorm(gated, os_, u, C, nw, Hd, 1e-6, gate_after=True)), n * inner * 8,
               "gated_group_rmsnorm")
        record(f"{label}.gated_group_rmsnorm", time_kernel(lambda: ops.gated_group_rmsnorm(gated, os_, u, C, nw, Hd, 1e-6)), n * inner * 8)
    logits = torch.randn(seqs, 32000, device=dev)
    record("decode.scale_softcap", time_kernel(lambda: ops.scale_softcap(logits, 0.5, 30.0)), seqs * 32000 * 8)
    return out


def pokadra_sizes(width, heads, kv_heads, dim, window, gru, ff, pz, vocab=32000):
    """A Pokadra model of eight layers (differential attention, minGRU, differential attention, minGRU, differential
    attention on the third layer's keys and values, minGRU, differential attention, minGRU) and the Pazenex configuration
    of the same width, feed-forward size, number of layer runs and window (``pz``: its attention and state-space sizes:
    twice the heads of half the size, since a differential head is two maps of ``dim`` over values of 2 ``dim``)."""
    def mlp():
        return {"kind": "dense", "ff": ff, "limit": 7.0}

    def att(kv_from=None):
        m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": 2 * dim, "scale": dim**-0.5, "diff": 0.8,
             "mask": {"size": window, "keep_first": 16},
             "rot": {"base": 1000000.0, "dims": dim, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "attention", "mlp": mlp(), "mixer": m}

    def rec():
        return {"type": "mingru", "mlp": mlp(), "mixer": {"width": gru}}

    pk = {"architecture": "Pokadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 4}, "residual_mult": 0.4,
          "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 36313, "mul_cur": 27191}}, "token_side": {"dim": 64},
          "layers": [att(), rec(), att(), rec(), att(kv_from=2), rec(), att(), rec()]}
    pazenex, _ = pazenex_sizes(width=width, heads=2 * heads, kv_heads=2 * kv_heads, dim=dim, ff=ff, vocab=vocab, **pz)
    for layer in pazenex["layers"]:
        if layer["type"] == "attention":
            layer["mixer"]["window"] = window
    return pk, pazenex


# a differential head of two maps of ``dim`` over values of 2 ``dim`` stands where two ordinary heads of ``dim`` stood;
# the minGRU is as wide as the Mamba-2 layer's inner size
POKADRA_SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=64, window=1024, gru=2048, ff=4096, pz=dict(ssm_heads=32, state=64, groups=4)),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=64, window=1024, gru=4096, ff=8192, pz=dict(ssm_heads=64, state=128, groups=8)),
    "w4096": dict(width=4096, heads=16, kv_heads=4, dim=128, window=1024, gru=8192, ff=14336, pz=dict(ssm_heads=128, state=128, groups=8)),
}


def pokadra_kernels(size, pk, tokens=4096, seqs=64):
    """Every kernel of the Pokadra parts beside the like kernel of the Pazenex parts, at one size: a prompt portion of
    ``tokens`` tokens and a decode step of ``seqs`` sequences at a context of 2,048 (both under the window of the size).  us,
    the bytes (or operations) the kernel has to move, and the share of the measured HBM peak (of the measured bf16 rate for
    attention over a portion)."""
    import torch

    from dli_b200.cache.pools import LayerCache
    from dli_b200.engine.batch import GroupView, StepBatch
    from dli_b200.kernels import attention as attn
    from dli_b200.kernels import ops

    dev, bf = "cuda", torch.bfloat16
    W, nh, nkv, d, ff, window, gru = size["width"], size["heads"], size["kv_heads"], size["dim"], size["ff"], size["window"], size["gru"]
    dv, page, side, vocab = 2 * d, 16, 64, 32000
    pz = size["pz"]
    out = {}

    def record(name, us, nbytes, like=None, flops=None):
        rec = {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        if flops is not None:
            rec["tflops_bf16"] = round(flops / us / 1e6, 1)
            rec["bf16_frac"] = round(flops / us / 1e6 / pk["bf16_tflops"], 3)
        if like:
            rec["like"] = like
        out[name] = rec

    for label, n, S in (("portion", tokens, 1), ("decode", seqs, seqs)):
        q_len = n // S
        context = tokens if S == 1 else 2048
        width = -(-context // page)
        tables = torch.arange(S * width, dtype=torch.int32, device=dev).view(S, width)
        q_start = torch.arange(S + 1, dtype=torch.int32, device=dev) * q_len
        kv_len = torch.full((S,), context, dtype=torch.int32, device=dev)
        seq_of = torch.repeat_interleave(torch.arange(S, dtype=torch.int32), q_len).to(dev)
        positions = (torch.arange(n, dtype=torch.int32) % q_len + (context - q_len)).to(dev)
        slots = (seq_of * width * page + positions).to(torch.int32)
        slot = torch.arange(S, dtype=torch.int32, device=dev)
        batch = StepBatch(n=n, num_seqs=S, num_single=S if q_len == 1 else 0, token_ids=positions, positions=positions, seq_of_token=seq_of,
                          q_start=q_start, kv_len=kv_len, state_slot=slot, logit_rows=positions[:0], groups=[GroupView(tables, slots)],
                          q_lens=[q_len] * S, starts=[context - q_len] * S, state_slots=list(range(S)), max_q_len=q_len, max_kv_len=context,
                          max_kv_len_single=context if q_len == 1 else 0)
        pages = S * width
        ids = torch.randint(0, vocab, (n,), dtype=torch.int32, device=dev)
        h = torch.randn(n, W, device=dev)
        a = torch.randn(n, W, device=dev).to(bf)
        w1, w2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
        y = torch.empty(n, W, dtype=bf, device=dev)
        # embedding with the hashed pair table
        table, pair = torch.randn(vocab, W, device=dev).to(bf), torch.randn(65522, W, device=dev).to(bf)
        prev = torch.zeros(S, dtype=torch.int32, device=dev)
        record(f"{label}.pair_embedding", time_kernel(lambda: ops.pair_embedding(h, table, 1.0, pair, 65521, 31, 17, ids, positions, seq_of, q_start, slot, prev, y)),
               n * W * 10, "embedding")
        record(f"{label}.embedding", time_kernel(lambda: ops.embedding(h, table, ids)), n * W * 6)
        # the norm behind a sublayer, added to the stream
        record(f"{label}.group_norm_add", time_kernel(lambda: ops.group_norm_add(h, a, w1, 4, 1e-6, 0.5, y)), n * W * 12, "post_add_layernorm")
        record(f"{label}.post_add_layernorm", time_kernel(lambda: ops.post_add_layernorm(y, h, a, w1, w2, 1e-6, 1e-6)), n * W * 12)
        # the token's own input: gate * table row
        g = torch.randn(n, side, device=dev).to(bf)
        side_table = torch.randn(vocab, 8 * side, device=dev).to(bf)
        record(f"{label}.gelu_mul_rows", time_kernel(lambda: ops.gelu_mul_rows(g, side_table, 3 * side, ids)), n * side * 6)
        # the mixture of the layers' results (the fifth layer's: six streams in, one out and its bfloat16 copy)
        hist = torch.randn(8, n, W, device=dev)
        dw = torch.full((9,), 0.2, device=dev)
        record(f"{label}.depth_average", time_kernel(lambda: ops.depth_average(hist[5], h, hist, dw, 6, y)), n * W * (6 * 4 + 4 + 2), "add_rmsnorm")
        record(f"{label}.add_rmsnorm", time_kernel(lambda: ops.add_rmsnorm(y, h, a, w1, 1e-6)), n * W * 12)
        # differential attention: preparation and attention, beside Pazenex's at twice the heads of half the size
        kp = torch.randn(pages + 1, nkv, page, 2 * d, device=dev).to(bf)
        vp = torch.randn(pages + 1, nkv, page, dv, device=dev).to(bf)
        cols = nh * 2 * d + nkv * (2 * d + dv) + nh
        proj = torch.randn(n, cols, device=dev).to(bf)
        q = torch.empty(n, nh * 2 * d, dtype=bf, device=dev)
        wn = torch.ones(d, device=dev)
        freq = (1.0 / (1000000.0 ** (torch.arange(0, d, 2).float() / d))).to(dev)
        moved = n * ((nh * 2 * d + nkv * (2 * d + dv)) * 4)
        record(f"{label}.diff_prep", time_kernel(lambda: ops.diff_prep(q, proj, nh * 2 * d, nh * 2 * d + nkv * 2 * d, wn, wn, 1e-6, positions, freq, 1.2, slots,
                                                                        kp, vp, nh, nkv, d, dv, d, page)), moved, "qk_norm_rotary_store")
        ph, pkv = 2 * nh, 2 * nkv
        kp2, vp2 = (torch.randn(pages + 1, pkv, page, d, device=dev).to(bf) for _ in range(2))
        proj2 = torch.randn(n, (ph + 2 * pkv) * d, device=dev).to(bf)
        wq2, wk2 = torch.ones(ph * d, device=dev), torch.ones(pkv * d, device=dev)
        record(f"{label}.qk_norm_rotary_store", time_kernel(lambda: ops.qk_norm_rotary_store(proj2, wq2, wk2, 1e-6, positions, freq, slots, kp2, vp2, ph, pkv, d, d, page,
                                                                                              values_from_keys=False)),
               n * (ph + 2 * pkv) * d * 4)
        att = torch.empty(n, nh * dv, dtype=bf, device=dev)
        keep = 16  # first tokens of a sequence that every window keeps
        gate = proj[:, cols - nh :]
        seen = sum(min(p + 1, window + keep) for p in range(context)) if S == 1 else float(min(context, window + keep))  # keys a token attends to
        kv_read = S * min(context, window + keep + (q_len if S == 1 else 0)) * nkv * (2 * d + dv) * 2
        us = time_kernel(lambda: attn.diff_attention(att, q, LayerCache(0, kp, vp, page), batch, gate, nh, d**-0.5, window, keep, 0.5, 0.2, 1e-6))
        record(f"{label}.diff_attention", us, kv_read + n * nh * (2 * d + dv) * 2, "sink_attention", flops=S * seen * nh * (4.0 * d + 4.0 * dv))
        pq, po = torch.randn(n, ph * d, device=dev).to(bf), torch.empty(n, ph * d, dtype=bf, device=dev)
        us = time_kernel(lambda: attn.paged_attention(po, pq, LayerCache(0, kp2, vp2, page), batch, ph, d**-0.5, window, sink=0.0))
        record(f"{label}.sink_attention", us, kv_read + n * ph * d * 4, flops=S * seen * ph * 4.0 * d)
        # the gate | up activation where it is a kernel of its own (9 to 511 tokens; otherwise it rides in the product's epilogue)
        gu = torch.randn(n, 2 * ff, device=dev).to(bf)
        act = torch.empty(n, ff, dtype=bf, device=dev)
        record(f"{label}.quick_gelu_bounded_mul", time_kernel(lambda: ops.silu_mul(act, gu, True, "quick_gelu", 7.0, 1.0)), n * ff * 6, "silu_mul")
        record(f"{label}.silu_mul", time_kernel(lambda: ops.silu_mul(act, gu, True)), n * ff * 6)
        # minGRU beside the Mamba-2 scan of the Pazenex model of this size
        p3 = torch.randn(n, 3 * gru, device=dev).to(bf)
        gs = torch.empty(n, gru, dtype=bf, device=dev)
        bz = torch.zeros(gru, device=dev)
        state = torch.zeros(S, gru, device=dev)
        us = time_kernel(lambda: ops.mingru_scan(gs, p3, bz, bz, state, q_start, slot, max_len=q_len))
        record(f"{label}.mingru_scan", us, n * gru * 8 + S * gru * 8, "ssm_scan")
        Hs, P, N, G = pz["ssm_heads"], 64, pz["state"], pz["groups"]
        sin, sC = Hs * P, Hs * P + 2 * G * N
        su = torch.randn(n, sin + sC + Hs, device=dev).to(bf)
        xbc = torch.randn(n, sC, device=dev).to(bf)
        sstate = torch.zeros(S, Hs, P, N, device=dev)
        ys = torch.empty(n, sin, device=dev)
        z3 = torch.zeros(Hs, device=dev)
        us = time_kernel(lambda: ops.ssm_scan(ys, xbc, su, sin + sC, z3, z3, z3 + 1, sstate, q_start, slot, G, max_len=q_len))
        record(f"{label}.ssm_scan", us, S * Hs * N * P * 8 + n * (sC * 2 + sin * 4))
    return out


def lokolorn_sizes(width, heads, kv_heads, dim, rec_heads, rec_dim, delta_heads, delta_kv_heads, delta_dim, rot_dim, kv_rank, window, ff, experts, top, sg,
                   vocab=32000):
    """A Lokolorn model of eight layer runs (attention and token-shift recurrence side by side, delta rule with a decay per channel,
    latent attention with a window and sinks, delta rule; the four run twice) whose routed feed-forward activates as many numbers a
    token as a dense one of size ``ff`` (``top`` experts of ff / top), and the Sugonex configuration of the same width, heads,
    feed-forward size and number of layer runs (``sg``: its sizes)."""
    def mlp():
        return {"kind": "moe", "expert": {"ff": ff // top}, "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}

    par = {"type": "parallel", "mlp": mlp(), "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": 4, "scale": 1.0, "rot": {"base": 10000.0, "dims": dim}},
        "right": {"heads": rec_heads, "dim": rec_dim, "decay_rank": 64}, "left_scale": 0.7, "right_scale": 0.7}}
    dl = {"type": "channel_delta", "mlp": mlp(), "mixer": {"heads": delta_heads, "kv_heads": delta_kv_heads, "dim": delta_dim, "vdim": delta_dim, "conv": 4,
                                                          "decay_rank": 64, "gate_rank": 64}}
    lat = {"type": "latent_attention", "mlp": mlp(), "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": dim, "kv_rank": kv_rank, "scale": (dim + rot_dim) ** -0.5, "mask": {"size": window},
        "rot": {"base": 500000.0, "dims": rot_dim, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}}
    lk = {"architecture": "Lokolorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [par, dl, lat, dl],
          "loop": {"start": 0, "stop": 4, "times": 2}}
    sugonex, _ = sugonex_sizes(width=width, ff=ff, vocab=vocab, **sg)
    return lk, sugonex


LOKOLORN_SIZES = {
    name: dict(width=s["width"], heads=s["heads"], kv_heads=s["pz"]["kv_heads"], dim=s["dim"], rec_heads=s["width"] // 64 // 2, rec_dim=64,
               delta_heads=s["delta_heads"], delta_kv_heads=s["delta_kv_heads"], delta_dim=s["delta_dim"], rot_dim=s["rot_dim"], kv_rank=s["kv_rank"],
               window=s["window"], ff=s["ff"], experts=16, top=4, sg={k: v for k, v in s.items() if k not in ("width", "ff")})
    for name, s in SUGONEX_SIZES.items()
}


def lokolorn_kernels(size, pk, tokens=4096, seqs=64):
    """Every kernel of the Lokolorn parts beside the like kernel of the Sugonex (or Llama) parts, at one size: a prompt portion of
    ``tokens`` tokens and a decode step of ``seqs`` sequences.  us, the bytes (or operations) the kernel has to move, and the share of
    the measured HBM peak (of the CUDA cores' float32 rate for the scans over a portion, of the measured bf16 rate for the products)."""
    import torch

    from dli_b200.kernels import gemm, ops

    dev, bf = "cuda", torch.bfloat16
    W, nh, nkv, d, ff = size["width"], size["heads"], size["kv_heads"], size["dim"], size["ff"]
    Hr, dr_ = size["rec_heads"], size["rec_dim"]
    Hd, Gd, dd = size["delta_heads"], size["delta_kv_heads"], size["delta_dim"]
    E, top = size["experts"], size["top"]
    eff = ff // top
    out = {}

    def record(name, us, nbytes, like=None, flops=None, tensor=False):
        rec = {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        if flops is not None and tensor:
            rec["tflops_bf16"] = round(flops / us / 1e6, 1)
            rec["bf16_frac"] = round(flops / us / 1e6 / pk["bf16_tflops"], 3)
        elif flops is not None:
            rec["tflops_fp32"] = round(flops / us / 1e6, 2)
            rec["simt_frac"] = round(flops / us / 1e6 / SIMT_FP32_TFLOPS, 3)
        if like:
            rec["like"] = like
        out[name] = rec

    for label, n, S in (("portion", tokens, 1), ("decode", seqs, seqs)):
        q_len = n // S
        q_start = torch.arange(S + 1, dtype=torch.int32, device=dev) * q_len
        seq_of = torch.repeat_interleave(torch.arange(S, dtype=torch.int32), q_len).to(dev)
        slot = torch.arange(S, dtype=torch.int32, device=dev)
        positions = (torch.arange(n, dtype=torch.int32) % q_len + (0 if S == 1 else 2048)).to(dev)
        # the norm that adds a scaled sublayer output (two terms, as behind a parallel mixer), beside the norm with two deltas
        h = torch.randn(n, W, device=dev)
        a, b = torch.randn(n, W, device=dev).to(bf), torch.randn(n, W, device=dev).to(bf)
        w1 = torch.ones(W, device=dev)
        y1, y2 = torch.empty(n, W, dtype=bf, device=dev), torch.empty(n, W, dtype=bf, device=dev)
        record(f"{label}.add_rmsnorm_scaled", time_kernel(lambda: ops.add_rmsnorm_scaled(y1, h, a, 0.7, b, 0.7, w1, w1, 1e-6)), n * W * 14, "add_rmsnorm_pair")
        record(f"{label}.add_rmsnorm_pair", time_kernel(lambda: ops.add_rmsnorm_pair(y1, y2, h, a, b, w1, w1, 1e-6)), n * W * 16)
        # loop entry and token shift
        table, ids = torch.randn(32000, W, device=dev).to(bf), torch.randint(0, 32000, (n,), dtype=torch.int32, device=dev)
        both = torch.empty(n, 2 * W, dtype=bf, device=dev)
        record(f"{label}.concat_stream_rows", time_kernel(lambda: ops.concat_stream_rows(both, h, table, ids)), n * W * 10)
        x = torch.randn(n, W, device=dev).to(bf)
        mu, shift = torch.rand(5, W, device=dev), torch.zeros(S, 1, W, dtype=bf, device=dev)
        blends = torch.empty(5, n, W, dtype=bf, device=dev)
        record(f"{label}.token_shift_blend", time_kernel(lambda: ops.token_shift_blend(blends, x, mu, shift, seq_of, q_start, slot)), n * W * 12)
        # attention half: convolution without activation, then rotation + unit RMS + pages
        C = (nh + 2 * nkv) * d
        u = torch.randn(n, C, device=dev).to(bf)
        mixed = torch.empty(n, C, dtype=bf, device=dev)
        cw, cstate = torch.randn(4, C, device=dev), torch.zeros(S, 3, C, dtype=bf, device=dev)
        record(f"{label}.causal_conv", time_kernel(lambda: ops.causal_conv_silu(mixed, u, 0, cw, None, cstate, seq_of, q_start, slot, activation=False)), n * C * 4,
               "causal_conv_silu")
        pages = n // 16 + S + 1
        kp, vp = (torch.zeros(pages, nkv, 16, d, dtype=bf, device=dev) for _ in range(2))
        slots = torch.arange(n, dtype=torch.int32, device=dev)
        inv = (1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))).to(dev)
        q = torch.empty(n, nh * d, dtype=bf, device=dev)
        record(f"{label}.rotary_unit_store", time_kernel(lambda: ops.rotary_unit_store(q, mixed, positions, inv, slots, kp, vp, nh, nkv, d, d, d, 1e-6, 16)),
               n * C * 4, "qk_norm_rotary_store")
        proj = torch.randn(n, (nh + 2 * nkv) * d, device=dev).to(bf)
        wq, wk = torch.ones(nh * d, device=dev), torch.ones(nkv * d, device=dev)
        record(f"{label}.qk_norm_rotary_store", time_kernel(lambda: ops.qk_norm_rotary_store(proj, wq, wk, 1e-6, positions, inv, slots, kp, vp, nh, nkv, d, d, 16,
                                                                                             True, False)), n * C * 4)
        # the two recurrences: float32 rows, then the walk; their like: the delta rule with one decay per head
        Ir = Hr * dr_
        rkvg, wz, w0 = torch.randn(4, n, Ir, device=dev).to(bf), torch.randn(n, Ir, device=dev).to(bf), torch.full((Ir,), -3.0, device=dev)
        rows = torch.empty(n, ops.decay_recurrence_row(Hr, Hr, dr_, dr_), device=dev)
        record(f"{label}.shift_decay_prep", time_kernel(lambda: ops.shift_decay_prep(rows, rkvg, wz, w0, Hr, dr_)), n * Ir * (8 + 16))
        st = torch.zeros(S, Hr, dr_, dr_, device=dev)
        o = torch.empty(n, Ir, device=dev)
        bonus = torch.randn(Hr, dr_, device=dev)
        us = time_kernel(lambda: ops.decay_recurrence(o, rows, st, q_start, slot, Hr, "bonus", bonus, max_len=q_len))
        record(f"{label}.recurrence_bonus", us, S * Hr * dr_ * dr_ * 8 + n * Ir * 20, "delta_rule_scan", flops=6.0 * n * Hr * dr_ * dr_)
        qk, inner = Gd * dd, Hd * dd
        qkv = torch.randn(n, 2 * qk + inner, device=dev).to(bf)
        uu = torch.randn(n, 2 * qk + inner + Hd + 128, device=dev).to(bf)
        aa, dtb, al = torch.randn(n, Hd * dd, device=dev).to(bf), torch.zeros(Hd * dd, device=dev), torch.full((Hd,), -3.0, device=dev)
        rows2 = torch.empty(n, ops.decay_recurrence_row(Gd, Hd, dd, dd), device=dev)
        record(f"{label}.channel_delta_prep", time_kernel(lambda: ops.channel_delta_prep(rows2, qkv, uu, 2 * qk + inner, aa, dtb, al, Hd, Gd, dd, dd, 1e-6)),
               n * (2 * qk + 2 * inner) * 6)
        st2 = torch.zeros(S, Hd, dd, dd, device=dev)
        o2 = torch.empty(n, inner, device=dev)
        us = time_kernel(lambda: ops.decay_recurrence(o2, rows2, st2, q_start, slot, Gd, "delta", None, max_len=q_len))
        record(f"{label}.recurrence_delta", us, S * Hd * dd * dd * 8 + n * (2 * qk + 2 * inner) * 4 + n * inner * 4, "delta_rule_scan", flops=8.0 * n * Hd * dd * dd)
        u3 = torch.randn(n, 2 * qk + 2 * inner + 2 * Hd, device=dev).to(bf)
        dt1, al1 = torch.zeros(Hd, device=dev), torch.full((Hd,), -3.0, device=dev)
        us = time_kernel(lambda: ops.delta_rule_scan(o2, qkv, u3, 2 * qk + 2 * inner, 2 * qk + 2 * inner + Hd, dt1, al1, st2, seq_of, q_start, slot, Gd, dd, 1e-6, max_len=q_len))
        record(f"{label}.delta_rule_scan", us, S * Hd * dd * dd * 8 + n * ((2 * qk + inner) * 2 + inner * 4), flops=8.0 * n * Hd * dd * dd)
        # routed feed-forward: router, experts; its like: the dense gated feed-forward of the same active size (library products + SiLU * up)
        router, corr = torch.randn(E, W, device=dev) * 0.05, torch.randn(E, device=dev) * 0.1
        ids2, wts = torch.empty(n, top, dtype=torch.int32, device=dev), torch.empty(n, top, device=dev)
        record(f"{label}.moe_route", time_kernel(lambda: ops.moe_route(ids2, wts, x, router, corr, 4, 2, 2.5)), n * W * 2 + E * W * 4)
        wgu, wd = (torch.randn(E, 2 * eff, W, device=dev) * 0.02).to(bf), (torch.randn(E, W, eff, device=dev) * 0.02).to(bf)
        y = torch.empty(n, W, dtype=bf, device=dev)
        flops = 6.0 * n * top * eff * W
        hit = min(E, n * top)
        record(f"{label}.moe_experts", time_kernel(lambda: ops.moe_experts(y, x, ids2, wts, wgu, wd, "silu")), hit * 3 * eff * W * 2 + n * W * 4, "dense_glu", flops=flops,
               tensor=True)
        dgu, ddn = (torch.randn(2 * ff, W, device=dev) * 0.02).to(bf), (torch.randn(W, ff, device=dev) * 0.02).to(bf)
        act = torch.empty(n, ff, dtype=bf, device=dev)

        def dense():
            ops.silu_mul(act, gemm.project(x, dgu), False)
            return gemm.project(act, ddn)

        record(f"{label}.dense_glu", time_kernel(dense), 3 * ff * W * 2 + n * W * 4, flops=6.0 * n * ff * W, tensor=True)
    return out


SIMT_FP32_TFLOPS = 148 * 128 * 2 * 1.9e9 / 1e12  # CUDA-core multiply-adds of a B200 at 1.9 GHz: the scan's ceiling (no float32 tensor-core path)


DESIGNS = {
    # design -> (sizes by name, what builds the two configurations of a size, the closest existing model, the kernels' table)
    "pazenex": (DESIGN_SIZES, pazenex_sizes, "llama", design_kernels),
    "sugonex": (SUGONEX_SIZES, sugonex_sizes, "pazenex", sugonex_kernels),
    "pokadra": (POKADRA_SIZES, pokadra_sizes, "pazenex", pokadra_kernels),
    "lokolorn": (LOKOLORN_SIZES, lokolorn_sizes, "sugonex", lokolorn_kernels),
}


def design_arm(args) -> int:
    """``--design NAME``: prefill and decode throughput of models of that architecture with random weights at layer sizes
    that resemble real models, beside the closest existing architecture at the same width, heads, feed-forward size and
    number of layer runs; and every kernel of the new parts beside its like among the other model's parts."""
    import torch

    import dli_b200

    sizes, build, other, kernels = DESIGNS[args.design]
    pk = peaks()
    line = {"design": args.design, "beside": other, "dtype": "bf16", "data": "synthetic: uniform-random token ids, seeded random weights", "sizes": {},
            "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "simt_fp32_tflops": round(SIMT_FP32_TFLOPS, 1), "source": pk["source"]}}
    names = [args.size] if args.size else list(sizes)
    for name in names:
        new_cfg, other_cfg = build(**sizes[name])
        # the matrix products' share of a prefill, counted on the Llama shape of these sizes
        flops_cfg = dict(LLAMA_3_2_1B, hidden_size=sizes[name]["width"], num_attention_heads=sizes[name]["heads"],
                         num_key_value_heads=sizes[name].get("kv_heads", sizes[name]["heads"]), head_dim=sizes[name]["dim"],
                         intermediate_size=sizes[name]["ff"], vocab_size=32000)
        rec = {}
        for label, cfg in ((args.design, new_cfg), (other, other_cfg)):
            model = dli_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            wbytes = all_weight_bytes(model)
            prefill = prefill_timed(model, flops_cfg, 8, pk["bf16_tflops"], reps=3, warmup=3, tokens=args.prompt_len)
            decode = decode_device_timed(model, args.batch, args.steps, args.warmup, blocks=1, prompt_len=args.prompt_len,
                                         context=args.prompt_len + 512)
            rec[label] = {"prefill_tok_s": round(prefill["value"], 1), "prefill_ms": round(prefill["ms"], 3),
                          "decode_tok_s": round(decode["tok_s"], 1), "decode_ms": round(decode["ms"], 4), "decode_launches": decode["launches"],
                          "weight_bytes": wbytes, "decode_weight_gb_s": round(wbytes / decode["ms"] / 1e6, 1)}
            del model
            torch.cuda.empty_cache()
        line["sizes"][name] = rec
    if not args.skip_points:
        line["kernels"] = kernels(sizes[args.size or "w2048"], pk)
    print(json.dumps(line))
    return 0


def config_record(cfg, layers, batch, source, extra=None):
    rec = {
        "model": "Llama-3.2-1B shape", "layers": layers, "layers_full": LLAMA_3_2_1B["num_hidden_layers"],
        "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
        "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
        "global_batch": batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "block_size": PAGE,
        "rope": "llama3 factor 32", "tied_embeddings": True, "parallelism": "1 GPU",
        "l2": "each step reads 2.5 GB of weights (> 126 MB L2); no flush", "peaks": source,
    }
    rec.update(extra or {})
    return rec


METRIC = "decode tok/s at batch {batch} (Llama-3.2-1B shape, random bf16 weights, context 2048..4096)"


# ----------------------------------------------------------------------------------------------
# The reference arm: the reference's own package and engine, nothing of this repository's.

def reference_unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def reference_engine(model, batch, attention):
    """The reference's engine as its own server builds it: LLMEngine.for_model with its graph shapes for the
    resolved decode kernel (src/dli/engine/engine.py:92-145, src/dli/server/__main__.py:138-175)."""
    from dli.engine import LLMEngine, SchedulerConfig
    from dli.engine.cuda_graph import default_shapes
    from dli.model import paged_attention

    kernel = paged_attention.resolve(attention, "cuda")
    pages = batch * (CONTEXT // PAGE) + 8
    pages += pages // 100 + 2  # its block manager holds one page in a hundred back at admission
    eng = LLMEngine.for_model(model, num_blocks=pages, block_size=PAGE, config=SchedulerConfig(max_num_seqs=max(batch, 1), max_num_batched_tokens=PROMPT_LEN),
                              enable_prefix_caching=False, cuda_graphs=default_shapes(kernel), decode_attention=kernel)
    return eng, kernel


def reference_decode(model, batch, steps, warmup, attention, clock=None):
    """Method of benchmarks/scripts/engine_profile.py:49-70 of the reference: requests of random ids
    ``randint(1000, vocab)``, steps until every prompt is computed, warm-up steps, then timed ``eng.step()`` loops
    around a synchronize; here in blocks of K steps, once by CUDA events and once by the host's clock."""
    import torch

    from dli.sampling import SamplingParams

    eng, kernel = reference_engine(model, batch, attention)
    vocab = model.config.vocab_size
    g = torch.Generator().manual_seed(2)
    for b in range(batch):
        eng.add_request(f"r{b}", torch.randint(1000, vocab, (PROMPT_LEN,), generator=g).tolist(),
                        SamplingParams(max_tokens=CONTEXT - PROMPT_LEN, ignore_eos=True))
    while any(r.num_computed_tokens < PROMPT_LEN for r in eng.scheduler.running + list(eng.scheduler.waiting)):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    blocks = max(1, timed_blocks(steps, warmup, 2560 - PROMPT_LEN) // 2)  # its widest graph holds 2,560 tokens
    if clock:
        clock.start()
    device_ms, host_ms = [], []
    for _ in range(blocks):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            assert len(eng.step()) == batch
        end.record()
        torch.cuda.synchronize()
        device_ms.append(start.elapsed_time(end) / steps)
    for _ in range(blocks):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            assert len(eng.step()) == batch
        torch.cuda.synchronize()
        host_ms.append((time.perf_counter() - t0) / steps * 1e3)
    if clock:
        clock.stop()
    ctx = statistics.mean(r.num_computed_tokens for r in eng.scheduler.running)
    graphs = getattr(eng.runner, "decode_graphs", None)
    summary = graphs.summary() if graphs is not None else None
    rows = next((g["batch"] for g in (summary or {}).get("graphs", []) if g["replays"]), batch)
    width = next((g["width_blocks"] for g in (summary or {}).get("graphs", []) if g["replays"]), -(-int(ctx) // PAGE))
    for rid in [r.request_id for r in eng.scheduler.running]:
        eng.abort(rid)
    del eng
    torch.cuda.empty_cache()
    return {"ms": statistics.median(device_ms), "host_ms": statistics.median(host_ms), "kernel": kernel, "mean_ctx": ctx,
            "graphs": None if summary is None else {"status": summary["status"], "replays": summary["replays"], "fallbacks": summary["fallbacks"]},
            "h2d": 8 * (4 * rows + rows * width), "d2h": 8 * batch}


def reference_prefill(model, attention, reps=3, warmup=2):
    """One prompt of 2,048 tokens as one step of the reference's engine (a pure prefill step as in
    benchmarks/scripts/pipeline_profile.py:60-103 of the reference)."""
    import torch

    from dli.sampling import SamplingParams

    eng, _ = reference_engine(model, 1, attention)
    g = torch.Generator().manual_seed(3)
    times = []
    for i in range(warmup + reps):
        eng.add_request(f"p{i}", torch.randint(1000, model.config.vocab_size, (PROMPT_LEN,), generator=g).tolist(), SamplingParams(max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = eng.step()
        end.record()
        torch.cuda.synchronize()
        assert len(out) == 1 and out[0].finished
        if i >= warmup:
            times.append(start.elapsed_time(end))
    del eng
    torch.cuda.empty_cache()
    return statistics.median(times)


def reference_arm(args) -> int:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "dli" / "engine" / "engine.py").exists():
        return reference_unavailable("no copy of the reference's package under baseline/_ref (its build backend, hatchling, is not installed, so pip "
                                     "cannot build it; a copy of its src/dli is what its pure wheel would install)")
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(ref))
    try:
        import torch

        from dli.model.config import ModelConfig
        from dli.model.llama import LlamaForCausalLM
    except Exception as exc:
        return reference_unavailable(f"the reference's package does not import here: {type(exc).__name__}: {exc}")
    if not torch.cuda.is_available():
        return reference_unavailable("no CUDA device")
    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=args.layers)
    pk = peaks()
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = LlamaForCausalLM(ModelConfig.from_hf_dict(cfg)).to(torch.bfloat16).eval()
    model.reset_rope(torch.device("cuda"))
    clocks = ClockSampler(device_id_for_smi())
    errors = []
    for attention in ("auto", "sdpa"):  # its Triton kernel first; should that not build or run on this GPU, its library attention
        try:
            with torch.inference_mode():
                main_run = reference_decode(model, args.batch, args.steps, args.warmup, attention, clocks)
                prefill_ms = reference_prefill(model, attention)
                points = {}
                if not args.skip_points:
                    for b in (1, 64):
                        run = reference_decode(model, b, args.steps, args.warmup, attention)
                        points[f"decode_b{b}"] = {"tok_s": round(b * 1000.0 / run["ms"], 1), "ms": round(run["ms"], 4),
                                                  "e2e_tok_s": round(b * 1000.0 / run["host_ms"], 1), "graphs": run["graphs"]}
            break
        except Exception as exc:  # noqa: BLE001 - whatever stops the reference is reported, not raised
            errors.append(f"decode_attention={attention}: {type(exc).__name__}: {exc}")
            clocks.stop()
            torch.cuda.synchronize()
    else:
        return reference_unavailable("the reference's engine does not run on this GPU: " + " | ".join(errors))
    weights = sum(p.numel() * p.element_size() for p in model.parameters())
    kv_token = 2 * args.layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    step_bytes = weights + args.batch * main_run["mean_ctx"] * kv_token
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    flops = prefill_flops(cfg, args.layers, PROMPT_LEN)
    line = {
        "metric": METRIC.format(batch=args.batch), "value": round(args.batch * 1000.0 / main_run["ms"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights (torch's default initialisation)",
        "impl": "reference",
        "config": config_record(cfg, args.layers, args.batch, pk["source"]),
        "e2e": {"value": round(args.batch * 1000.0 / main_run["host_ms"], 2), "unit": "tokens/s", "h2d_bytes_per_step": main_run["h2d"],
                "d2h_bytes_per_step": main_run["d2h"], "ms_per_step": round(main_run["host_ms"], 4)},
        "prefill": {"value": round(PROMPT_LEN * 1000.0 / prefill_ms, 1), "tokens": PROMPT_LEN, "ms": round(prefill_ms, 4),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "flops": flops, "unit": "tokens/s"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "reference": {"decode_attention": main_run["kernel"], "cuda_graphs": main_run["graphs"], "earlier_errors": errors,
                      "path": "LLMEngine.for_model / add_request / step of the unmodified package under baseline/_ref"},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=LLAMA_3_2_1B["num_hidden_layers"], help="fewer layers than the model has, if memory or time needs it")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the main batch size (for profiling runs)")
    ap.add_argument("--skip-more", action="store_true", help="leave out the other shapes and contexts (the \"more\" key)")
    ap.add_argument("--phase", default="all", choices=["all", "decode", "prefill", "sample"],
                    help="profiling runs: only the device-timed decode steps, only the prefill step, or only the sampling kernel (prints a short line)")
    ap.add_argument("--no-graphs", action="store_true", help="profiling runs: launch the step's kernels one by one")
    ap.add_argument("--design", default=None, choices=["pazenex", "sugonex", "pokadra", "lokolorn"],
                    help="another measurement: this architecture beside Llama at equal sizes, and its kernels beside their likes (prints its own line)")
    ap.add_argument("--size", default=None, choices=list(DESIGN_SIZES), help="--design: one size only (every design has these names)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                    help="profiling runs: the context at which decoding starts (--phase decode), the prompt's length (--phase prefill)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)
    if args.design:
        return design_arm(args)

    import torch

    import dli_b200
    from dli_b200.kernels import ops  # noqa: F401

    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=args.layers)
    pk = peaks()
    if args.phase == "sample":
        print(json.dumps({"phase": "sample", "vocab": cfg["vocab_size"], "unit": "us", **sampling_timed(cfg["vocab_size"])}))
        return 0
    model = dli_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    clocks = ClockSampler(device_id_for_smi())
    if args.phase == "decode":
        run = decode_device_timed(model, args.batch, args.steps, args.warmup, graphs=not args.no_graphs, blocks=1, prompt_len=args.prompt_len,
                                  context=max(CONTEXT, args.prompt_len + 512))
        print(json.dumps({"phase": "decode", "batch": args.batch, "layers": args.layers, "prompt_len": args.prompt_len, **run}))
        return 0
    if args.phase == "prefill":
        print(json.dumps({"phase": "prefill", "layers": args.layers, "graphs": not args.no_graphs,
                          **prefill_timed(model, cfg, args.layers, pk["bf16_tflops"], reps=args.steps, warmup=args.warmup, tokens=args.prompt_len,
                                          graphs=not args.no_graphs)}))
        return 0
    main_run = decode_device_timed(model, args.batch, args.steps, args.warmup, clocks)
    clocks.start()  # the end-to-end steps are timed too: keep sampling
    e2e = decode_end_to_end(model, args.batch, args.steps, args.warmup)
    clocks.stop()
    prefill = prefill_timed(model, cfg, args.layers, pk["bf16_tflops"])
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = decode_point(model, b, args.steps, args.warmup, pk["hbm_gbs"])

    step_bytes = weight_bytes(model) + args.batch * main_run["mean_ctx"] * cache_bytes_per_token(model)
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": METRIC.format(batch=args.batch),
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, seeded random weights", "impl": "ours",
        "config": config_record(cfg, args.layers, args.batch, pk["source"]),
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "timed_blocks": {"blocks": main_run["blocks"], "ms_per_step": main_run["block_ms"], "reported": "median"},
        "prefill": {k: (round(v, 4) if isinstance(v, float) else v) for k, v in prefill.items()},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "clocks": clocks.summary(),
    }
    if not args.skip_more and args.layers == LLAMA_3_2_1B["num_hidden_layers"]:
        line["more"] = more_points(model, args.steps, args.warmup, pk)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
