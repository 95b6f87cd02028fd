#!/usr/bin/env python
"""Headline benchmark: Llama-2-7B nf4 weight-only, batch-1 greedy decode tok/s (BASELINE.json configs[1]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one decode token.  `value` = tokens/s over K replays of the captured decode graph with everything
resident in HBM (CUDA events, max over ranks); `e2e` = the same metric through the public `generate()` call with the
prompt in pinned HOST memory and the tokens read back to the host inside the timed region.  N > 1 = the same model
tensor-parallel over N GPUs (strong scaling), launched by torchrun.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (config name, quantize mode, batch, prompt tokens, context pre-fill)
    "llama2-7b-nf4-bs1": ("Llama-2-7b-hf", "nf4", 1, 16, 0),
    "llama2-7b-nf4-bs1-ctx2048": ("Llama-2-7b-hf", "nf4", 1, 16, 2032),
    "llama2-13b-int4-bs1-ctx2048": ("Llama-2-13b-hf", "int4", 1, 16, 2032),
    "llama2-13b-int4-bs4-ctx2048": ("Llama-2-13b-hf", "int4", 4, 16, 2032),
    "llama2-13b-int4-bs16-ctx2048": ("Llama-2-13b-hf", "int4", 16, 16, 2032),
    "mistral-7b-int4-bs1-ctx3936": ("Mistral-7B-v0.1", "int4", 1, 16, 3920),  # block_size 4096 bounds prompt + steps
    "mistral-7b-int4-bs1": ("Mistral-7B-v0.1", "int4", 1, 16, 0),
    "llama2-70b-int4-bs1-ctx2048": ("Llama-2-70b-hf", "int4", 1, 16, 2032),
}
# algorithmic bytes per parameter: nf4 / fp4 = 4 bits + one fp32 absmax per 64; int4 g128 = 4 bits + one fp16 scale and
# one 4-bit zero-point per 128 (0.51953).  The kernels stream the fused half2 {scale, zero} form of int4 (0.53125): reported as
# `streamed_bytes_per_param`, not used for the roofline fraction.
BPP = {"nf4": 0.5 + 4 / 64, "fp4": 0.5 + 4 / 64, "int4": 0.5 + 2.5 / 128}
BPP_STREAMED = {"nf4": 0.5 + 4 / 64, "fp4": 0.5 + 4 / 64, "int4": 0.5 + 4 / 128}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler(threading.Thread):
    """SM clock + throttle reasons sampled in-process through NVML every ~2 ms (B200_PROFILING.md clocks line); only the
    samples taken between mark_start() and mark_end() -- the timed region -- are reported."""

    def __init__(self, device: "torch.device"):
        super().__init__(daemon=True)
        self.rows, self._stop_evt, self.t0, self.t1, self.handle, self.nv = [], threading.Event(), None, None, None, None
        try:
            import pynvml as nv

            nv.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            try:
                self.handle = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.handle = nv.nvmlDeviceGetHandleByIndex(device.index or 0)
            self.nv = nv
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001
            self.err = str(e)

    def run(self):
        nv = self.nv
        if nv is None:
            return
        while not self._stop_evt.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.rows.append((time.perf_counter(), float(mhz), int(reasons)))
            except Exception:
                pass
            time.sleep(0.002)

    def mark_start(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=1.0)
        nv = self.nv
        if nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": "nvml unavailable: " + getattr(self, "err", "?")}
        rows = [r for r in self.rows if self.t0 is not None and self.t0 <= r[0] <= (self.t1 or 1e99)]
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4,
                "hw_power_brake_slowdown": 0x80}
        mask = 0
        for r in rows:
            mask |= r[2]
        return {"sm_mhz": statistics.median([r[1] for r in rows]) if rows else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for n, b in bits.items() if mask & b), "samples": len(rows),
                "source": "NVML in-process, 2 ms period, samples inside the timed region only"}


def build_random_model(cfg_name: str, mode: str, max_seq: int, batch: int, fabric, n_layer=None):
    """Random-init weights of the named architecture (N(0, 0.02), seed 1234, bf16), materialised one matrix at a
    time on the GPU, sharded in full precision (generate/tp.py order) and then quantized by the library."""
    from lit_gpt_b200 import GPT, Config, QLinear
    from lit_gpt_b200.generate.tp import shard_lm_head, tensor_parallel

    kw = {} if n_layer is None else {"n_layer": n_layer}
    cfg = Config.from_name(cfg_name, **kw)
    full = Config.from_name(cfg_name, **kw)
    with fabric._precision.module_init_context(), torch.device("meta"):
        model = GPT(cfg)
    full_shapes = {n: (m.out_features, m.in_features) for n, m in model.named_modules() if isinstance(m, QLinear)}
    styles = {}
    if fabric.world_size > 1:
        model = tensor_parallel(fabric, model)
        if os.environ.get("B200_TP_SHARD_LM_HEAD", "1") == "1":   # §8f-3: vocabulary slices per rank, all-gathered over peer memory
            model = shard_lm_head(fabric, model)
        for n in full_shapes:
            styles[n] = 0 if n.endswith(("attn.attn", "fc_1", "fc_2", "fc")) else (1 if n.endswith("proj") else None)
        if getattr(model, "lm_head_sharded", False):
            styles["lm_head"] = 0
    dev = fabric.device
    gen = torch.Generator(device=dev)
    for i, (name, mod) in enumerate(model.named_modules()):
        if isinstance(mod, QLinear):
            gen.manual_seed(1234 + i)
            w = torch.empty(full_shapes[name], dtype=torch.bfloat16, device=dev).normal_(0.0, 0.02, generator=gen)
            if styles.get(name) is not None:
                w = torch.tensor_split(w, fabric.world_size, dim=styles[name])[fabric.global_rank].contiguous()
            mod.weight = torch.nn.Parameter(w, requires_grad=False)
            mod.quantize_()
            del w
        elif isinstance(mod, torch.nn.Embedding):
            gen.manual_seed(1234 + i)
            mod.weight = torch.nn.Parameter(torch.empty(mod.weight.shape, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.02, generator=gen), requires_grad=False)
        elif type(mod).__name__ == "RMSNorm":
            mod.weight = torch.nn.Parameter(torch.ones(mod.weight.shape, dtype=torch.bfloat16, device=dev), requires_grad=False)
    with fabric.init_tensor():
        model.max_seq_length = max_seq
        model.cos, model.sin = model.rope_cache()
        model.set_kv_cache(batch_size=batch)
    model.eval()
    return model, full


def step_bytes(full_cfg, mode: str, ctx: int, batch: int, tp: int, head_sharded: bool = False) -> dict:
    """Algorithmic HBM bytes of one decode step per GPU: packed weights + scales of every Linear once,
    plus the filled KV rows at n_query_groups heads in bf16.  lm_head is replicated under TP (generate/tp.py:77-80)."""
    c = full_cfg
    per_layer = c.n_embd * (c.n_head + 2 * c.n_query_groups) * c.head_size + c.n_embd * c.n_embd + 3 * c.n_embd * c.intermediate_size
    head = c.padded_vocab_size * c.n_embd
    w = (c.n_layer * per_layer / tp + head / (tp if head_sharded else 1)) * BPP[mode]
    kv = 2 * c.n_layer * c.n_query_groups * c.head_size * 2 * ctx * batch / tp
    return {"weights": w, "kv": kv, "total": w + kv}


def gemv_only_step(model, x, y_attn, xn=None):
    """Exactly the dequant-GEMV launches of one fused decode step (norm prologues, residual / SwiGLU epilogues
    included), without attention / embedding / argmax: used to time the dominant kernel in isolation.
    xn: the pre-normalised rows for batches above model.SPLIT_NORM_ROWS, where the step runs RMSNorm as its own launch and the
    GEMVs take plain rows (GPT._fused_decode): the same launches as the step's, the norm launches themselves left out."""
    from lit_gpt_b200 import kernels as K

    eps = model.config.norm_eps

    def lin(q, inp, nxt=None, **kw):
        return q.gemv(inp, prefetch=None if nxt is None else nxt.tiled, **kw)

    def normed(q, inp, w, nxt=None, **kw):
        if xn is not None:
            return lin(q, xn, nxt, **kw)
        return lin(q, inp, nxt, norm_weight=w, norm_eps=eps, **kw)

    blocks = list(model.transformer.h)
    for li, block in enumerate(blocks):
        a, m = block.attn, block.mlp
        nxt_qkv = blocks[li + 1].attn.attn if li + 1 < len(blocks) else model.lm_head
        normed(a.attn, x, block.norm_1.weight, a.proj)
        if model.tp_world_size > 1:
            h = lin(a.proj, y_attn, m.fc_1)
            act = lin(m.fc_1, x, m.proj, other=m.fc_2, delta=h, norm_weight=block.norm_2.weight, norm_eps=eps)
            lin(m.proj, act, nxt_qkv)
        else:
            x2 = lin(a.proj, y_attn, m.fc_1, residual=x)
            act = normed(m.fc_1, x2, block.norm_2.weight, m.proj, other=m.fc_2)
            lin(m.proj, act, nxt_qkv, residual=x2)
    normed(model.lm_head, x, model.transformer.ln_f.weight, blocks[0].attn.attn)


def time_graph(graph, n: int, world: int) -> float:
    """ms for n replays, CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks."""
    import torch.distributed as dist

    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
    return float(ms.item())


def cpu_reference_sample(cfg_name: str, steps: int, layers: int = 4, warmup: int = 0) -> dict:
    """The reference's CPU path (generate/base.py on the host cores, fp32) restated by oracle/model_ref.py, on a
    BOUNDED sample: `layers` of the model's blocks at full width + the full lm_head, extrapolated to full depth."""
    from lit_gpt_b200 import Config
    from oracle import model_ref as M

    torch.set_num_threads(os.cpu_count() or 1)
    cfg = Config.from_name(cfg_name)
    rc = M.RefConfig.from_any(Config.from_name(cfg_name, n_layer=layers))
    g = torch.Generator().manual_seed(1234)
    p = {}
    shapes = {"attn.attn": ((cfg.n_head + 2 * cfg.n_query_groups) * cfg.head_size, cfg.n_embd), "attn.proj": (cfg.n_embd, cfg.n_embd),
              "mlp.fc_1": (cfg.intermediate_size, cfg.n_embd), "mlp.fc_2": (cfg.intermediate_size, cfg.n_embd),
              "mlp.proj": (cfg.n_embd, cfg.intermediate_size)}
    for i in range(layers):
        for k, s in shapes.items():
            p[f"transformer.h.{i}.{k}.weight"] = torch.empty(s).normal_(0, 0.02, generator=g)
        p[f"transformer.h.{i}.norm_1.weight"] = torch.ones(cfg.n_embd)
        p[f"transformer.h.{i}.norm_2.weight"] = torch.ones(cfg.n_embd)
    p["transformer.ln_f.weight"] = torch.ones(cfg.n_embd)
    p["transformer.wte.weight"] = torch.empty(cfg.padded_vocab_size, cfg.n_embd).normal_(0, 0.02, generator=g)
    p["lm_head.weight"] = torch.empty(cfg.padded_vocab_size, cfg.n_embd).normal_(0, 0.02, generator=g)
    T = 16
    st = M.RefState(rc, T + steps + warmup + 2, 1, torch.float32, pos_dtype=torch.float32)
    prompt = torch.randint(0, cfg.vocab_size, (T,), generator=g)
    with torch.inference_mode():
        logits = M.gpt_forward(rc, p, prompt.view(1, -1), torch.arange(T), st)
        tok = M.sample(logits, 0.0)
        # head-only time (ln_f + lm_head) to extrapolate depth correctly
        x = torch.randn(1, 1, cfg.n_embd)
        t0 = time.perf_counter()
        for _ in range(2):
            M.linear(M.rmsnorm(x, p["transformer.ln_f.weight"], cfg.norm_eps), p["lm_head.weight"])
        t_head = (time.perf_counter() - t0) / 2
        for i in range(warmup):
            logits = M.gpt_forward(rc, p, tok.view(1, 1), torch.tensor([T + i]), st)
            tok = M.sample(logits, 0.0)
        t0 = time.perf_counter()
        for i in range(steps):
            logits = M.gpt_forward(rc, p, tok.view(1, 1), torch.tensor([T + warmup + i]), st)
            tok = M.sample(logits, 0.0)
        t_step = (time.perf_counter() - t0) / steps
    full = layers >= cfg.n_layer
    t_full = t_step if full else (t_step - t_head) * cfg.n_layer / layers + t_head
    depth = "all blocks (full depth, nothing extrapolated)" if full else \
        f"{layers} of {cfg.n_layer} blocks at full width + full lm_head, extrapolated to full depth ({t_full * 1e3:.1f} ms/token)"
    return {"value": 1.0 / t_full, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port", "steps_timed": steps,
            "timed_s": t_step * steps,
            "sample": f"oracle/model_ref.py generate loop (reference generate/base.py restated), fp32, {depth}; "
                      f"{steps} decode tokens timed after a {T}-token prompt and {warmup} warm-up tokens; "
                      f"measured {t_step * 1e3:.1f} ms/token"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cfg_name, mode, batch, T, ctx = WORKLOADS[args.workload]
    from lit_gpt_b200 import Config

    # exactly `--steps` decode tokens are timed after `--warmup` untimed ones.  Full depth when the host has the memory for
    # the fp32 weights (7B: 27 GB) and the run stays within minutes; else a 4-block sample at full width, extrapolated
    # (stated in cpu_baseline.sample either way).
    cfg = Config.from_name(cfg_name)
    per_layer = cfg.n_embd * (cfg.n_head + 2 * cfg.n_query_groups) * cfg.head_size + cfg.n_embd * cfg.n_embd + 3 * cfg.n_embd * cfg.intermediate_size
    need = 4 * (cfg.n_layer * per_layer + 2 * cfg.padded_vocab_size * cfg.n_embd)
    try:
        import psutil

        avail = psutil.virtual_memory().available
    except Exception:
        avail = 0
    full_depth = avail > need * 1.3 and args.steps + args.warmup <= 64 and os.environ.get("B200_REF_SAMPLE", "0") != "1"
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    cb = cpu_reference_sample(cfg_name, steps, layers=cfg.n_layer if full_depth else 4, warmup=max(0, args.warmup))
    line = {
        "impl": "reference", "metric": "Llama-2-7B nf4 decode tok/s (bs=1)", "value": cb["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 / cb["value"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "note": "reference CPU path (bitsandbytes has no CPU nf4: fp32 weights)"},
        "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    import torch.distributed as dist

    import lit_gpt_b200.generate.base as gb
    from lit_gpt_b200 import QuantPrecision
    from lit_gpt_b200 import kernels as K
    from lit_gpt_b200.fabric import Fabric

    if not torch.cuda.is_available():
        raise SystemExit("bench.py (impl ours) needs a CUDA device: the product path has no CPU fallback")
    if os.environ.get("B200_TUNE_OCC"):  # development: A/B switches of b200_qgemv_tiled_tune (e.g. 14 = no K / V cache L2 hint)
        K.qgemv_tiled_tune(0, int(os.environ["B200_TUNE_OCC"]), False)
    cfg_name, mode, batch, T, ctx = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    fabric = Fabric(devices="auto", strategy="ddp" if world > 1 else None, plugins=QuantPrecision(mode, torch.bfloat16))
    fabric.launch()
    rank = fabric.global_rank
    K_steps, W = args.steps, max(args.warmup, 3)
    max_seq = ctx + T + W + K_steps + 2
    t_build = time.perf_counter()
    model, full_cfg = build_random_model(cfg_name, mode, max_seq, batch, fabric, n_layer=args.layers)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    assert model.fused_decode_ready(), "model is not on the fused CUDA path"
    dev = fabric.device
    g = torch.Generator().manual_seed(1234)
    prompt_host = torch.randint(0, full_cfg.vocab_size, (T,), generator=g).pin_memory()

    def prefill_context():
        for blk in model.transformer.h:
            blk.attn.kv_cache.reset_parameters()
        if ctx:  # synthetic N(0,1) K/V history, then the prompt after it
            gg = torch.Generator(device=dev).manual_seed(7)
            for blk in model.transformer.h:
                blk.attn.kv_cache.k[:, :, :ctx].normal_(generator=gg)
                blk.attn.kv_cache.v[:, :, :ctx].normal_(generator=gg)

    # ---- device-resident timing: K replays of the captured decode step --------------------------------------
    prefill_context()
    prompt = prompt_host.to(dev, non_blocking=True)
    tok = gb.next_token(model, torch.arange(ctx, ctx + T, device=dev), prompt.view(1, -1).expand(batch, -1).contiguous(), temperature=0.0)
    dg = gb.DecodeGraph(model, 0.0, None, torch.int64)
    if batch > 1:
        dg.token = torch.zeros(batch, dtype=torch.int64, device=dev)
        dg._step = lambda: K.argmax_(model(dg.token.view(batch, 1), dg.pos), dg.token, pos_inout=dg.pos)
    dg.token.copy_(tok.expand(batch) if batch > 1 else tok)
    dg.pos.fill_(ctx + T)
    n0 = K.launch_count()
    dg._step()
    launches_per_step = K.launch_count() - n0
    dg.pos.fill_(ctx + T)
    dg.capture()
    sampler = ClockSampler(dev)
    if rank == 0:
        sampler.start()   # running through the warm-up so that the first timed step is already covered
    time_graph(dg.graph, W, world)
    sampler.mark_start()
    ms = time_graph(dg.graph, K_steps, world)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else {}
    tok_s = batch * K_steps / (ms / 1e3)
    ctx_mid = ctx + T + W + K_steps // 2
    bytes_step = step_bytes(full_cfg, mode, ctx_mid, batch, world, bool(getattr(model, "lm_head_sharded", False)))

    # ---- dominant kernel in isolation: the dequant-GEMV launches of one step, same weights (3.7 GB >> L2) ----
    x = torch.randn(batch, model.transformer.wte.weight.shape[1], device=dev).to(torch.bfloat16)
    y_attn = torch.randn(batch, model.transformer.h[0].attn.proj.in_features, device=dev).to(torch.bfloat16)
    from lit_gpt_b200.model import SPLIT_NORM_ROWS

    split_norm = batch > SPLIT_NORM_ROWS and world == 1   # the step then normalises in its own launch and the GEMVs take plain rows
    xn = K.rmsnorm(x, model.transformer.ln_f.weight, model.config.norm_eps) if split_norm else None
    n0 = K.launch_count()
    gemv_only_step(model, x, y_attn, xn)
    gemv_launches = K.launch_count() - n0
    gg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gg):
        gemv_only_step(model, x, y_attn, xn)
    time_graph(gg, W, 1)
    reps = max(8, min(K_steps, 64))
    gemv_ms = time_graph(gg, reps, 1) / reps
    peaks, peak_src = measured_peaks()
    achieved = bytes_step["weights"] / (gemv_ms / 1e3) / 1e9
    # dram__bytes_read + dram__bytes_write per launch from the committed ncu capture of this workload (ratio to the
    # algorithmic bytes, measured per layer shape); null for workloads that were not captured
    traffic = None
    tpath = os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles", "r02_traffic.json")
    if not os.path.exists(tpath):
        tpath = os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles", "r01_traffic.json")
    if os.path.exists(tpath):
        tj = json.load(open(tpath))
        if tj.get("workload") == args.workload and world == 1:
            traffic = tj["traffic_over_algorithmic"] * bytes_step["weights"] / max(1, gemv_launches)
    kernel_name = "qgemv_v4_kernel" if batch == 1 or world > 1 else ("qgemv_nb_kernel" if split_norm else "qgemv_v4_kernel (norm-fused launches) + qgemv_nb_kernel (plain rows)")
    roofline = {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                "traffic_source": None if traffic is None else "constant: ncu dram__bytes_read+write of the committed capture (profiles/), "
                                                                "scaled by this run's algorithmic bytes; not measured by this run",
                "peak_source": peak_src, "streamed_bytes_per_param": BPP_STREAMED[mode],
                "launches_per_step": gemv_launches, "avg_launch_us": gemv_ms * 1e3 / max(1, gemv_launches),
                "algorithmic_bytes_per_launch": bytes_step["weights"] / max(1, gemv_launches),
                "whole_step_frac": bytes_step["total"] / (ms / K_steps / 1e3) / 1e9 / peaks["hbm_gbs"],
                "frac_of_nominal_8TBs": achieved / 8000.0}

    # ---- end to end through generate(): pinned host prompt -> H2D -> prefill + K tokens -> D2H ------------------
    e2e = None
    if batch == 1 and ctx == 0:  # generate() starts at position 0: long-context points report the device number only
        prefill_context()
        n_total = T + K_steps
        gb.generate(model, prompt_host.to(dev), min(n_total, T + 4), temperature=0.0, eos_id=-1)  # warm
        prefill_context()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        out = gb.generate(model, prompt_host.to(dev, non_blocking=True), n_total, temperature=0.0, eos_id=-1)
        out_host = out.cpu()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        e_ms = torch.tensor([max(e0.elapsed_time(e1), wall * 1e3)], device=dev)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        new = out_host.numel() - T
        polls = -(-max(new - 1, 1) // gb.EOS_POLL)
        e2e = {"value": new / (float(e_ms.item()) / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": T * 8 / new,
               "d2h_bytes_per_step": (out_host.numel() * 8 + polls * (new // 2) * 8) / new,
               "note": f"generate(): {T}-token prompt from pinned host memory, prefill + {new} greedy tokens, EOS polled on the "
                       f"host every {gb.EOS_POLL} tokens, sequence copied back; includes python + launch overhead"}

    if rank != 0:
        return
    cb = None
    if world == 1 and not args.no_cpu_baseline:
        cb = cpu_reference_sample(cfg_name, 4)
    line = {
        "metric": "Llama-2-7B nf4 decode tok/s (bs=1)" if args.workload == "llama2-7b-nf4-bs1" else f"{args.workload} decode tok/s",
        "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": K_steps, "warmup": W, "ms_per_step": ms / K_steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "model": cfg_name, "quantize": mode, "batch": batch, "prompt_tokens": T,
                   "context_prefill": ctx, "max_seq": max_seq, "parallelism": f"tp{world}", "lm_head_sharded": bool(getattr(model, "lm_head_sharded", False)), "n_layer": full_cfg.n_layer,
                   "l2_policy": "weights per step (>= 0.4 GB/GPU) exceed the 126 MB L2; no flush needed",
                   "bytes_per_step": bytes_step, "build_s": round(t_build, 1)},
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches_per_step * K_steps), "launches_per_step": int(launches_per_step),
        "roofline": roofline, "cpu_baseline": cb,
        "hbm_frac_of_measured_whole_step": roofline["whole_step_frac"],
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# --compare pomipel: the Pomipel design beside the closest existing model (a Llama-shaped GPT in unquantized bf16) at equal
# width, heads, head size, layers and feed-forward FLOPs per token; random weights.  Prints one JSON line of its own kind.
# ---------------------------------------------------------------------------------------------------------
ARCH_SIZES = {
    # name: width, heads, head size, kv_rank, q_rank, experts, top, expert ff
    "w1024": (1024, 8, 128, 256, 512, 16, 4, 512),
    "w2048": (2048, 16, 128, 512, 1024, 32, 4, 1024),
    "w4096": (4096, 32, 128, 512, 1536, 64, 6, 1024),
}


def _timed(fn, iters: int, flush) -> float:
    """Mean device time of fn() in ms over `iters` calls, L2 flushed (a write larger than L2) before each timed call."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def _graphed(step):
    """step() captured in a CUDA graph (after two warm-up runs); falls back to the eager callable."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step(); step()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        return g.replay, True
    except Exception:
        torch.cuda.synchronize()
        return step, False


def run_arch_compare(args) -> None:
    from lit_gpt_b200 import GPT, Config
    from lit_gpt_b200 import kernels as K
    from lit_gpt_b200.config import LatentMixerSpec, LayerSpec, MoESpec, PomipelConfig
    from lit_gpt_b200.pomipel import Pomipel

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, peak_source = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    n_layer, vocab, T, ctx = 4, 32000, args.prompt, args.prompt
    iters = max(3, min(args.steps, 20))
    launches0 = K.launch_count()
    out = {}
    for name in (args.sizes.split(",") if args.sizes else ARCH_SIZES):
        d, H, hs, r, qr, E, top, ff = ARCH_SIZES[name]
        inter = (2 * top * ff // 3 + 63) // 64 * 64     # three matrices against two: equal feed-forward FLOPs per token
        layers = [LayerSpec("latent_attention", LatentMixerSpec(H, hs, hs, r, qr, hs ** -0.5, None if i % 2 == 0 else i - 1),
                            MoESpec(E, top, ff, 4, 2)) for i in range(n_layer)]
        pom = Pomipel(PomipelConfig(vocab_size=vocab, n_embd=d, block_size=ctx + 64, embedding_scale=d ** 0.5, logit_scale=1.0, layers=layers))
        pom = pom.to(dev).to(torch.bfloat16).eval()
        pom.reset_parameters()
        gpt = GPT(Config(name="bench", block_size=ctx + 64, vocab_size=vocab, padding_multiple=64, n_layer=n_layer, n_head=H, n_embd=d,
                         rotary_percentage=1.0, parallel_residual=False, bias=False, _norm_class="RMSNorm", _mlp_class="LLaMAMLP",
                         intermediate_size=inter))
        gpt.apply(gpt._init_weights)
        gpt = gpt.to(dev).to(torch.bfloat16).eval()
        res = {"gpt_intermediate": inter}
        with torch.inference_mode():
            for label, model in (("pomipel", pom), ("gpt", gpt)):
                for B in (1, 8):
                    if label == "gpt":
                        model.set_kv_cache(batch_size=B, device=dev, dtype=torch.bfloat16)
                    else:
                        model.set_kv_cache(batch_size=B)
                    idx = torch.randint(0, vocab, (B, T), device=dev)
                    pos = torch.arange(T, device=dev)
                    if B == 1:
                        ms = _timed(lambda: model(idx, pos), iters, flush)
                        res[f"{label}_prefill_tok_s"] = round(T / ms * 1e3)
                    else:
                        model(idx, pos)
                    tok, p1 = idx[:, :1].contiguous(), torch.tensor([T], device=dev)
                    step, graphed = _graphed(lambda: model(tok, p1))
                    ms = _timed(step, iters, flush)
                    res[f"{label}_decode_b{B}_tok_s"] = round(B / ms * 1e3)
                    res[f"{label}_decode_b{B}_graphed"] = graphed
                    del step
                model.clear_kv_cache()
            # like kernels alone, with their algorithmic work against the measured peaks
            kern = {}
            q = torch.randn(T, H * hs, device=dev, dtype=torch.bfloat16)
            kv = torch.randn(T, 2 * H * hs, device=dev, dtype=torch.bfloat16)
            seqs = torch.tensor([[0, T, 0, 0]], dtype=torch.int32, device=dev)
            att_flops = 4.0 * H * hs * T * (T + 1) / 2
            ms = _timed(lambda: K.latent_prefill(q, kv[:, : H * hs], kv[:, H * hs :], seqs, T, H, hs, hs, hs ** -0.5), iters, flush)
            kern["prefill_attention_pomipel"] = {"ms": ms, "frac_of_measured_bf16": att_flops / (ms * 1e-3) / tf}
            q4 = torch.randn(1, H, T, hs, device=dev, dtype=torch.bfloat16)
            kc = torch.randn(1, H, T, hs, device=dev, dtype=torch.bfloat16)
            vc = torch.randn(1, H, T, hs, device=dev, dtype=torch.bfloat16)
            pos = torch.arange(T, device=dev)
            ms = _timed(lambda: K.attn_prefill(q4, kc, vc, pos), iters, flush)
            kern["prefill_attention_gpt"] = {"ms": ms, "frac_of_measured_bf16": att_flops / (ms * 1e-3) / tf}
            B = 8
            mx = pom.blocks[0].mixer
            cache = torch.randn(B, ctx, r, device=dev, dtype=torch.bfloat16)
            qd = torch.randn(B, H * hs, device=dev, dtype=torch.bfloat16)
            slot = torch.arange(B, dtype=torch.int32, device=dev)
            rp = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
            from lit_gpt_b200.latent import decode_splits
            ms = _timed(lambda: K.latent_decode(qd, mx.w_uk, mx.w_uv, cache, slot, rp, H, hs, hs, hs ** -0.5, decode_splits(ctx, B * (-(-H // 16)))), iters, flush)
            roof = max(B * ctx * r * 2 / hbm, 4.0 * B * H * ctx * r / tf)
            kern["decode_attention_pomipel"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3),
                                                "bytes": B * ctx * r * 2, "flops": 4.0 * B * H * ctx * r}
            kc8 = torch.randn(B, H, ctx, hs, device=dev, dtype=torch.bfloat16)
            vc8 = torch.randn(B, H, ctx, hs, device=dev, dtype=torch.bfloat16)
            qkv = torch.randn(B, 3 * H * hs, device=dev, dtype=torch.bfloat16)
            p1 = torch.tensor([ctx - 1], device=dev)
            ms = _timed(lambda: K.attn_decode(qkv, gpt.cos, gpt.sin, p1, kc8, vc8, H, H, hs, hs), iters, flush)
            roof = 2.0 * B * H * ctx * hs * 2 / hbm
            kern["decode_attention_gpt"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3),
                                            "bytes": 2.0 * B * H * ctx * hs * 2}
            x = torch.randn(T, d, device=dev, dtype=torch.bfloat16)
            ms = _timed(lambda: pom.blocks[0].mlp(x), iters, flush)
            # bytes: every expert's two matrices once (T * top >= E: all are touched), the gathered rows, the hidden rows and the
            # per-choice outputs each written and read back; the dense layer below: three matrices and its own intermediates
            moe_bytes = 2.0 * E * ff * d * 2 + T * top * (2 * d * 2 + 4 * ff * 2 + 2 * d * 2) + 2 * T * d * 2
            roof = max(4.0 * T * top * ff * d / tf, moe_bytes / hbm)
            kern["feed_forward_pomipel"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * T * top * ff * d / (ms * 1e-3) / tf,
                                            "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": moe_bytes}
            x3 = x.view(1, T, d)
            ms = _timed(lambda: gpt.transformer.h[0].mlp(x3), iters, flush)
            mlp_bytes = 3.0 * inter * d * 2 + T * (2 * d * 2 + 5 * inter * 2)
            roof = max(6.0 * T * inter * d / tf, mlp_bytes / hbm)
            kern["feed_forward_gpt"] = {"ms": ms, "frac_of_measured_bf16": 6.0 * T * inter * d / (ms * 1e-3) / tf,
                                        "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": mlp_bytes}
            xs, act, w0 = torch.randn(T, d, device=dev), torch.empty(T, d, device=dev, dtype=torch.bfloat16), pom.blocks[0].norm_1
            ms = _timed(lambda: K.residual_norm_add(x, w0, 1e-5, xs, act), iters, flush)
            kern["residual_norm_pomipel"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            so = torch.empty_like(x)
            ms = _timed(lambda: K.rmsnorm(x, gpt.transformer.h[0].norm_1.weight, 1e-5, delta=x, sum_out=so), iters, flush)
            kern["residual_norm_gpt"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 2 + 2 + 2) / (ms * 1e-3) / hbm}
            res["kernels"] = {k: {a: (round(b, 4) if isinstance(b, float) else b) for a, b in v.items()} for k, v in kern.items()}
        out[name] = res
        del pom, gpt
        torch.cuda.empty_cache()
    print(json.dumps({"compare": "pomipel", "layers": n_layer, "prompt": T, "context": ctx, "dtype": "bf16", "data": "synthetic, random weights",
                      "l2": "flushed between timed calls", "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                                                                       "source": peak_source},
                      "gpu_launches": int(K.launch_count() - launches0), "sizes": out}), flush=True)


# ---------------------------------------------------------------------------------------------------------
# --compare lefalix: the Lefalix design beside the closest existing model (Pomipel: the other slot-served design with an fp32
# residual stream and sparse experts) at equal width, heads, head size, layers and expert sizes; random weights.
# ---------------------------------------------------------------------------------------------------------
LEFALIX_SIZES = {
    # name: width, heads, key-value heads, head size, window, low rank, experts, top, expert ff, dense ff
    "w1024": (1024, 8, 2, 128, 512, 64, 16, 4, 512, 4096),
    "w2048": (2048, 16, 4, 128, 1024, 128, 32, 4, 1024, 8192),
    "w4096": (4096, 32, 8, 128, 1024, 128, 64, 6, 1024, 14336),
}


def run_lefalix_compare(args) -> None:
    from lit_gpt_b200 import kernels as K
    from lit_gpt_b200.config import (DeltaMixerSpec, DenseMLPSpec, GatedMoESpec, LatentMixerSpec, LayerSpec, LefalixConfig, LefalixLayerSpec, MoESpec,
                                     ParallelMixerSpec, PomipelConfig, RotarySpec, WindowMixerSpec)
    from lit_gpt_b200.latent import decode_splits
    from lit_gpt_b200.lefalix import Lefalix
    from lit_gpt_b200.pomipel import Pomipel
    from lit_gpt_b200.ragged import state_batch

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, peak_source = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    vocab, T = 32000, args.prompt
    iters = max(3, min(args.steps, 20))
    launches0 = K.launch_count()
    bf = torch.bfloat16
    out = {}
    for name in (args.sizes.split(",") if args.sizes else LEFALIX_SIZES):
        d, H, G, hs, W, rank, E, top, ff, dff = LEFALIX_SIZES[name]
        rot = RotarySpec(dims=hs // 2, base=1e6, factor=4.0, original=4096.0, fast=32.0, slow=1.0)

        def par(mlp):
            return LefalixLayerSpec("parallel", ParallelMixerSpec(WindowMixerSpec(H, G, hs, hs, 4, W, hs ** -0.5, rot), DeltaMixerSpec(H // 2, H // 4, hs, hs, 4)), mlp)

        def chan(mlp):
            return LefalixLayerSpec("channel_delta", DeltaMixerSpec(H, H // 2, hs, hs, 4, True, rank, rank), mlp)

        layers = [chan(DenseMLPSpec(dff)), par(GatedMoESpec(E, top, ff, 4, 2)), par(DenseMLPSpec(dff)), chan(GatedMoESpec(E, top, ff, 4, 2))]
        lef = Lefalix(LefalixConfig(vocab_size=vocab, n_embd=d, layers=layers)).to(dev).to(bf).eval()
        lef.reset_parameters()
        lef.max_seq_length = T + 64
        players = [LayerSpec("latent_attention", LatentMixerSpec(H, hs, hs, 4 * hs, 8 * hs, hs ** -0.5, None if i % 2 == 0 else i - 1),
                             MoESpec(E, top, ff, 4, 2)) for i in range(4)]
        pom = Pomipel(PomipelConfig(vocab_size=vocab, n_embd=d, block_size=T + 64, embedding_scale=d ** 0.5, logit_scale=1.0, layers=players))
        pom = pom.to(dev).to(bf).eval()
        pom.reset_parameters()
        res = {}
        with torch.inference_mode():
            for label, model in (("lefalix", lef), ("pomipel", pom)):
                for B in (1, 8):
                    model.set_kv_cache(batch_size=B)
                    idx = torch.randint(0, vocab, (B, T), device=dev)
                    pos = torch.arange(T, device=dev)
                    if B == 1:
                        ms = _timed(lambda: model(idx, pos), iters, flush)
                        res[f"{label}_prefill_tok_s"] = round(T / ms * 1e3)
                    else:
                        model(idx, pos)
                    tok, p1 = idx[:, :1].contiguous(), torch.tensor([T], device=dev)
                    step, graphed = _graphed(lambda: model(tok, p1))
                    ms = _timed(step, iters, flush)
                    res[f"{label}_decode_b{B}_tok_s"] = round(B / ms * 1e3)
                    res[f"{label}_decode_b{B}_graphed"] = graphed
                    del step
                model.clear_kv_cache()
            kern = {}
            # prefill attention: both designs on the same tensor-core tiles; the window's work is T * W - W^2 / 2 score pairs
            q = torch.randn(T, H * hs, device=dev, dtype=bf)
            kv = torch.randn(T, 2 * G * hs, device=dev, dtype=bf)
            sink = torch.zeros(H, device=dev, dtype=bf)
            batch, _ = state_batch([(0, 0, T)], dev)
            kr, vr = torch.zeros(1, W, G * hs, device=dev, dtype=bf), torch.zeros(1, W, G * hs, device=dev, dtype=bf)
            pairs = sum(min(i + 1, W) for i in range(T))
            ms = _timed(lambda: K.window_attn(q, kv[:, : G * hs], kv[:, G * hs :], kr, vr, sink, batch.seq_state, batch.row_seq, T, H, G, hs, hs, W,
                                              hs ** -0.5, from_start=True), iters, flush)
            kern["prefill_attention_lefalix"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * H * hs * pairs / (ms * 1e-3) / tf, "includes": "ring store"}
            kvp = torch.randn(T, 2 * H * hs, device=dev, dtype=bf)
            seqs = torch.tensor([[0, T, 0, 0]], dtype=torch.int32, device=dev)
            ms = _timed(lambda: K.latent_prefill(q, kvp[:, : H * hs], kvp[:, H * hs :], seqs, T, H, hs, hs, hs ** -0.5), iters, flush)
            kern["prefill_attention_pomipel"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * H * hs * T * (T + 1) / 2 / (ms * 1e-3) / tf}
            # decode attention: bytes that must come from HBM
            B = 8
            qd, kd = torch.randn(B, H * hs, device=dev, dtype=bf), torch.randn(B, 2 * G * hs, device=dev, dtype=bf)
            krb, vrb = torch.randn(B, W, G * hs, device=dev, dtype=bf), torch.randn(B, W, G * hs, device=dev, dtype=bf)
            bd, _ = state_batch([(b, T, 1) for b in range(B)], dev)
            ms = _timed(lambda: K.window_attn(qd, kd[:, : G * hs], kd[:, G * hs :], krb, vrb, sink, bd.seq_state, bd.row_seq, 1, H, G, hs, hs, W,
                                              hs ** -0.5), iters, flush)
            roof = 2.0 * B * G * W * hs * 2 / hbm
            kern["decode_attention_lefalix"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": 2.0 * B * G * W * hs * 2,
                                                "includes": "ring store"}
            r = 4 * hs
            mx = pom.blocks[0].mixer
            cache = torch.randn(B, T, r, device=dev, dtype=bf)
            slot = torch.arange(B, dtype=torch.int32, device=dev)
            rp = torch.full((B,), T - 1, dtype=torch.int32, device=dev)
            ms = _timed(lambda: K.latent_decode(qd, mx.w_uk, mx.w_uv, cache, slot, rp, H, hs, hs, hs ** -0.5, decode_splits(T, B * (-(-H // 16)))), iters, flush)
            roof = max(B * T * r * 2 / hbm, 4.0 * B * H * T * r / tf)
            kern["decode_attention_pomipel"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": B * T * r * 2}
            # the recurrence: prompts are bound by the chain of T dependent state updates, single tokens by the state's bytes
            dm = lef.blocks[0].mixer
            Hd, Gd = dm.spec.heads, dm.spec.kv_heads
            floats = Hd * K.delta_rule_state_floats(hs, hs)
            for label, ch in (("channel", True), ("head", False)):
                qf, kf, vf = torch.randn(T, Gd * hs, device=dev), torch.randn(T, Gd * hs, device=dev), torch.randn(T, Hd * hs, device=dev)
                be, de = torch.randn(T, Hd, device=dev, dtype=bf), torch.randn(T, Hd * hs if ch else Hd, device=dev, dtype=bf)
                al, db = torch.zeros(Hd, device=dev, dtype=bf), torch.zeros(Hd * hs if ch else Hd, device=dev, dtype=bf)
                st1 = torch.zeros(1, floats, device=dev)
                ms = _timed(lambda: K.delta_rule(qf, kf, vf, be, de, al, db, st1, batch.seq_state, Hd, Gd, hs, hs, ch, max_rows=T), iters, flush)
                kern[f"delta_rule_prompt_{label}_decay"] = {"ms": ms, "us_per_token": ms * 1e3 / T, "fp32_tflops": 6.0 * T * Hd * hs * hs / (ms * 1e-3) / 1e12}
                st8 = torch.zeros(B, floats, device=dev)
                ms = _timed(lambda: K.delta_rule(qf[:B], kf[:B], vf[:B], be[:B], de[:B], al, db, st8, bd.seq_state, Hd, Gd, hs, hs, ch), iters, flush)
                roof = 2.0 * B * floats * 4 / hbm
                kern[f"delta_rule_decode_{label}_decay"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": 2.0 * B * floats * 4}
            # short convolution with rotation and norm (reads bf16 rows, writes bf16 rows) beside Pomipel's norm of projected rows
            wm = lef.blocks[1].mixer.left
            cols = wm.cols
            qkv, dst = torch.randn(T, cols, device=dev, dtype=bf), torch.empty(T, cols, device=dev, dtype=bf)
            tail = torch.zeros(1, 3, cols, device=dev, dtype=bf)
            fr = wm.inv_freq(dev)
            groups = [K.conv_group(wm.conv[: H * hs], dst[:, : H * hs], 0, H, hs, post=1, rot_dims=hs // 2, inv_freq=fr, rot_mscale=rot.magnitude, eps=1e-5),
                      K.conv_group(wm.conv[H * hs : (H + G) * hs], dst[:, H * hs : (H + G) * hs], H * hs, G, hs, post=1, rot_dims=hs // 2, inv_freq=fr,
                                   rot_mscale=rot.magnitude, eps=1e-5),
                      K.conv_group(wm.conv[(H + G) * hs :], dst[:, (H + G) * hs :], (H + G) * hs, G, hs)]
            ms = _timed(lambda: K.short_conv(qkv, groups, 4, tail, batch.seq_state, batch.row_seq), iters, flush)
            kern["short_conv_rotate_norm_lefalix"] = {"ms": ms, "frac_of_measured_hbm": T * cols * 4.0 / (ms * 1e-3) / hbm}
            down, cq = torch.randn(T, cols, device=dev, dtype=bf), torch.empty(T, cols, device=dev, dtype=bf)
            wn = torch.ones(cols, device=dev, dtype=bf)
            ms = _timed(lambda: K.rms_rows(T, 1e-5, K.rms_seg(down, wn, cq, cols, False), in_dtype=bf, out_dtype=bf, device=dev), iters, flush)
            kern["norm_of_projected_rows_pomipel"] = {"ms": ms, "frac_of_measured_hbm": T * cols * 4.0 / (ms * 1e-3) / hbm}
            # residual kernels
            x = torch.randn(T, d, device=dev, dtype=bf)
            x2 = torch.randn(T, d, device=dev, dtype=bf)
            xs, act = torch.randn(T, d, device=dev), torch.empty(T, d, device=dev, dtype=bf)
            blk = lef.blocks[1]
            ms = _timed(lambda: K.sandwich_residual(xs, x, blk.norm_1b, 1e-5, w0=blk.mixer.left_out, y1=x2, w1=blk.mixer.right_out, pre_w=blk.norm_2, act=act),
                        iters, flush)
            kern["residual_two_branches_lefalix"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.sandwich_residual(xs, x, blk.norm_2b, 1e-5, pre_w=blk.norm_1, act=act), iters, flush)
            kern["residual_one_branch_lefalix"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.residual_norm_add(x, pom.blocks[0].norm_1, 1e-5, xs, act), iters, flush)
            kern["residual_norm_pomipel"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            # feed-forwards over T tokens
            ms = _timed(lambda: lef.blocks[1].mlp(x), iters, flush)
            kern["experts_lefalix"] = {"ms": ms, "frac_of_measured_bf16": 6.0 * T * top * ff * d / (ms * 1e-3) / tf}
            ms = _timed(lambda: pom.blocks[0].mlp(x), iters, flush)
            kern["experts_pomipel"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * T * top * ff * d / (ms * 1e-3) / tf}
            ms = _timed(lambda: lef.blocks[0].mlp(x), iters, flush)
            kern["dense_mlp_lefalix"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * T * dff * d / (ms * 1e-3) / tf}
            res["kernels"] = {k: {a: (round(b, 4) if isinstance(b, float) else b) for a, b in v.items()} for k, v in kern.items()}
        out[name] = res
        del lef, pom
        torch.cuda.empty_cache()
    print(json.dumps({"compare": "lefalix", "layers": 4, "prompt": T, "context": T, "dtype": "bf16", "data": "synthetic, random weights",
                      "l2": "flushed between timed calls", "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                                                                       "source": peak_source},
                      "gpu_launches": int(K.launch_count() - launches0), "sizes": out}), flush=True)


# ---------------------------------------------------------------------------------------------------------
# --compare nulezen: the Nulezen design beside the closest existing model (Lefalix: the other design with sliding-window attention
# over key / value rings, gated experts and an fp32 residual stream) at equal width, heads, head size, window, layers and expert
# sizes; random weights.
# ---------------------------------------------------------------------------------------------------------
def run_nulezen_compare(args) -> None:
    from lit_gpt_b200 import kernels as K
    from lit_gpt_b200.config import (ClampedMoESpec, DeltaMixerSpec, DenseMLPSpec, GatedMoESpec, GatedWindowSpec, LefalixConfig, LefalixLayerSpec,
                                     NulezenConfig, NulezenLayerSpec, ParallelMixerSpec, RotarySpec, WindowMixerSpec)
    from lit_gpt_b200.lefalix import Lefalix
    from lit_gpt_b200.nulezen import Nulezen
    from lit_gpt_b200.ragged import state_batch

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, peak_source = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    vocab, T = 32000, args.prompt
    iters = max(3, min(args.steps, 20))
    launches0 = K.launch_count()
    bf = torch.bfloat16
    out = {}
    for name in (args.sizes.split(",") if args.sizes else LEFALIX_SIZES):
        d, H, G, hs, W, rank, E, top, ff, dff = LEFALIX_SIZES[name]

        def first(mlp):
            return NulezenLayerSpec("attention", GatedWindowSpec(H, G, hs, hs, W, hs ** -0.5, distance=True, gate="element"), mlp)

        def second(mlp):
            return NulezenLayerSpec("attention_2", GatedWindowSpec(H, G, hs, hs, W, hs ** -0.5, rot=RotarySpec(dims=hs, base=1e6, interleaved=False),
                                                                   bias=True, gate="head"), mlp)

        def experts():
            return ClampedMoESpec(E, top, ff, 7.0, shared_ff=ff, shared_limit=7.0)

        nul = Nulezen(NulezenConfig(vocab_size=vocab, n_embd=d, embedding_scale=1.0, logit_scale=1.0, loop_start=0, loop_stop=2, loop_times=2,
                                    layers=[first(DenseMLPSpec(dff)), second(experts())])).to(dev).to(bf).eval()   # two layers run twice: four layer runs
        nul.reset_parameters()
        nul.max_seq_length = T + 64
        rot = RotarySpec(dims=hs // 2, base=1e6, factor=4.0, original=4096.0, fast=32.0, slow=1.0)

        def par(mlp):
            return LefalixLayerSpec("parallel", ParallelMixerSpec(WindowMixerSpec(H, G, hs, hs, 4, W, hs ** -0.5, rot), DeltaMixerSpec(H // 2, H // 4, hs, hs, 4)), mlp)

        lef = Lefalix(LefalixConfig(vocab_size=vocab, n_embd=d, layers=[par(DenseMLPSpec(dff)), par(GatedMoESpec(E, top, ff, 4, 2)),
                                                                        par(DenseMLPSpec(dff)), par(GatedMoESpec(E, top, ff, 4, 2))])).to(dev).to(bf).eval()
        lef.reset_parameters()
        lef.max_seq_length = T + 64
        res = {}
        with torch.inference_mode():
            for label, model in (("nulezen", nul), ("lefalix", lef)):
                for B in (1, 8):
                    model.set_kv_cache(batch_size=B)
                    idx = torch.randint(0, vocab, (B, T), device=dev)
                    pos = torch.arange(T, device=dev)
                    if B == 1:
                        ms = _timed(lambda: model(idx, pos), iters, flush)
                        res[f"{label}_prefill_tok_s"] = round(T / ms * 1e3)
                    else:
                        model(idx, pos)
                    tok, p1 = idx[:, :1].contiguous(), torch.tensor([T], device=dev)
                    step, graphed = _graphed(lambda: model(tok, p1))
                    ms = _timed(step, iters, flush)
                    res[f"{label}_decode_b{B}_tok_s"] = round(B / ms * 1e3)
                    res[f"{label}_decode_b{B}_graphed"] = graphed
                    del step
                model.clear_kv_cache()
            kern = {}
            # prefill attention: both designs on the same tensor-core tiles; the window's work is T * W - W^2 / 2 score pairs
            q = torch.randn(T, H * hs, device=dev, dtype=bf)
            kv = torch.randn(T, 2 * G * hs, device=dev, dtype=bf)
            sink = torch.zeros(H, device=dev, dtype=bf)
            r1, r2 = torch.full((H,), 0.5, device=dev, dtype=bf), torch.ones(H, device=dev, dtype=bf)
            gate_e, gate_h = torch.randn(T, H * hs, device=dev, dtype=bf), torch.randn(T, H, device=dev, dtype=bf)
            batch, _ = state_batch([(0, 0, T)], dev, positions=True)
            kr, vr = torch.zeros(1, W, G * hs, device=dev, dtype=bf), torch.zeros(1, W, G * hs, device=dev, dtype=bf)
            pairs = sum(min(i + 1, W) for i in range(T))
            kk, vv = kv[:, : G * hs], kv[:, G * hs :]

            def win(qq, k_, v_, b, rows, **kw):
                return K.window_attn(qq, k_, v_, kr if rows > 1 else krb, vr if rows > 1 else vrb, kw.pop("sink", None), b.seq_state, b.row_seq, rows, H, G,
                                     hs, hs, W, hs ** -0.5, from_start=rows > 1, **kw)

            for label, kw in (("nulezen_distance_bias_gate_per_number", dict(dist=(r1, r2), gate=gate_e)),
                              ("nulezen_gate_per_head", dict(gate=gate_h, gate_per_head=True)), ("lefalix_sink", dict(sink=sink))):
                ms = _timed(lambda: win(q, kk, vv, batch, T, **dict(kw)), iters, flush)
                kern[f"prefill_attention_{label}"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * H * hs * pairs / (ms * 1e-3) / tf, "includes": "ring store"}
            # decode attention: bytes that must come from HBM
            B = 8
            qd, kd = torch.randn(B, H * hs, device=dev, dtype=bf), torch.randn(B, 2 * G * hs, device=dev, dtype=bf)
            krb, vrb = torch.randn(B, W, G * hs, device=dev, dtype=bf), torch.randn(B, W, G * hs, device=dev, dtype=bf)
            bd, _ = state_batch([(b, T, 1) for b in range(B)], dev, positions=True)
            roof = 2.0 * B * G * W * hs * 2 / hbm
            for label, kw in (("nulezen_distance_bias_gate_per_number", dict(dist=(r1, r2), gate=gate_e[:B])),
                              ("nulezen_gate_per_head", dict(gate=gate_h[:B], gate_per_head=True)), ("lefalix_sink", dict(sink=sink))):
                ms = _timed(lambda: win(qd, kd[:, : G * hs], kd[:, G * hs :], bd, 1, **dict(kw)), iters, flush)
                kern[f"decode_attention_{label}"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": 2.0 * B * G * W * hs * 2,
                                                     "includes": "ring store"}
            # rotation of q and k in place beside Lefalix's convolution + rotation + norm (both read and write each projected number once)
            nm = nul.blocks[1].mixer
            proj = torch.randn(T, nm.cols, device=dev, dtype=bf)
            fr = nm.freq(dev)
            qv, kv_ = proj[:, : H * hs], proj[:, H * hs : (H + G) * hs]
            ms = _timed(lambda: K.head_rope(T, batch.row_pos, 0.0, K.rope_seg(qv, qv, H, hs, freq=fr, rot_dims=hs, interleaved=False),
                                            K.rope_seg(kv_, kv_, G, hs, freq=fr, rot_dims=hs, interleaved=False), dtype=bf, device=dev), iters, flush)
            kern["rotation_nulezen"] = {"ms": ms, "frac_of_measured_hbm": T * (H + G) * hs * 4.0 / (ms * 1e-3) / hbm}
            wm = lef.blocks[1].mixer.left
            cols = wm.cols
            qkv, dst = torch.randn(T, cols, device=dev, dtype=bf), torch.empty(T, cols, device=dev, dtype=bf)
            tail = torch.zeros(1, 3, cols, device=dev, dtype=bf)
            fl = wm.inv_freq(dev)
            groups = [K.conv_group(wm.conv[: H * hs], dst[:, : H * hs], 0, H, hs, post=1, rot_dims=hs // 2, inv_freq=fl, rot_mscale=rot.magnitude, eps=1e-5),
                      K.conv_group(wm.conv[H * hs : (H + G) * hs], dst[:, H * hs : (H + G) * hs], H * hs, G, hs, post=1, rot_dims=hs // 2, inv_freq=fl,
                                   rot_mscale=rot.magnitude, eps=1e-5),
                      K.conv_group(wm.conv[(H + G) * hs :], dst[:, (H + G) * hs :], (H + G) * hs, G, hs)]
            ms = _timed(lambda: K.short_conv(qkv, groups, 4, tail, batch.seq_state, batch.row_seq), iters, flush)
            kern["short_conv_rotate_norm_lefalix"] = {"ms": ms, "frac_of_measured_hbm": T * cols * 4.0 / (ms * 1e-3) / hbm}
            # residual kernels
            x, x2, x3 = (torch.randn(T, d, device=dev, dtype=bf) for _ in range(3))
            xs, act = torch.randn(T, d, device=dev), torch.empty(T, d, device=dev, dtype=bf)
            nb_, lb = nul.blocks[1], lef.blocks[1]
            ms = _timed(lambda: K.scaled_residual(xs, y0=x, s0=nb_.ls1, y1=x2, y2=x3, s1=nb_.ls2, norm=nb_.norm.terms(), act=act), iters, flush)
            kern["residual_three_branches_norm_nulezen"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 2 + 2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.scaled_residual(xs, y0=x, s0=nb_.ls1, y1=x2, s1=nb_.ls2, norm=nb_.norm.terms(), act=act), iters, flush)
            kern["residual_two_branches_norm_nulezen"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.sandwich_residual(xs, x, lb.norm_1b, 1e-5, w0=lb.mixer.left_out, y1=x2, w1=lb.mixer.right_out, pre_w=lb.norm_2, act=act),
                        iters, flush)
            kern["residual_two_branches_lefalix"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            # feed-forwards over T tokens
            ms = _timed(lambda: nb_.mlp(x), iters, flush)
            kern["experts_nulezen"] = {"ms": ms, "frac_of_measured_bf16": 6.0 * T * top * ff * d / (ms * 1e-3) / tf}
            ms = _timed(lambda: lb.mlp(x), iters, flush)
            kern["experts_lefalix"] = {"ms": ms, "frac_of_measured_bf16": 6.0 * T * top * ff * d / (ms * 1e-3) / tf}
            ms = _timed(lambda: nb_.mlp.shared(x), iters, flush)
            kern["shared_expert_nulezen"] = {"ms": ms, "frac_of_measured_bf16": 6.0 * T * ff * d / (ms * 1e-3) / tf}
            ms = _timed(lambda: nul.blocks[0].mlp(x), iters, flush)
            kern["dense_mlp_xielu_nulezen"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * T * dff * d / (ms * 1e-3) / tf}
            ms = _timed(lambda: lef.blocks[0].mlp(x), iters, flush)
            kern["dense_mlp_gelu_lefalix"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * T * dff * d / (ms * 1e-3) / tf}
            # the activations alone (bytes read and written once)
            hid, both = torch.randn(T, dff, device=dev, dtype=bf), torch.randn(T * top, 2 * ff, device=dev, dtype=bf)
            ms = _timed(lambda: K.xielu_(hid, nul.blocks[0].mlp.act), iters, flush)
            kern["xielu_nulezen"] = {"ms": ms, "frac_of_measured_hbm": T * dff * 4.0 / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.activation_(hid, K.ACT_GELU), iters, flush)
            kern["gelu_lefalix"] = {"ms": ms, "frac_of_measured_hbm": T * dff * 4.0 / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.glu_clamped(both, 7.0, 1.702), iters, flush)
            kern["clamped_gate_nulezen"] = {"ms": ms, "frac_of_measured_hbm": T * top * ff * 6.0 / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.glu(both, K.ACT_SILU), iters, flush)
            kern["silu_gate_lefalix"] = {"ms": ms, "frac_of_measured_hbm": T * top * ff * 6.0 / (ms * 1e-3) / hbm}
            # routers (one CTA per token; reads the token and the router's rows)
            ms = _timed(lambda: nb_.mlp.router(x), iters, flush)
            kern["router_nulezen"] = {"ms": ms, "us_per_token": ms * 1e3 / T}
            ms = _timed(lambda: lb.mlp.router(x), iters, flush)
            kern["router_lefalix"] = {"ms": ms, "us_per_token": ms * 1e3 / T}
            res["kernels"] = {k: {a: (round(b, 4) if isinstance(b, float) else b) for a, b in v.items()} for k, v in kern.items()}
        out[name] = res
        del nul, lef
        torch.cuda.empty_cache()
    print(json.dumps({"compare": "nulezen", "layers": 4, "prompt": T, "context": T, "dtype": "bf16", "data": "synthetic, random weights",
                      "l2": "flushed between timed calls", "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                                                                       "source": peak_source},
                      "gpu_launches": int(K.launch_count() - launches0), "sizes": out}), flush=True)


# ---------------------------------------------------------------------------------------------------------
# --compare fizadra: the Fizadra design beside the closest existing model (Pomipel: the other design with latent attention over an
# fp32 residual stream) at equal width, heads, head size, latent size and layers; random weights.
# ---------------------------------------------------------------------------------------------------------
FIZADRA_SIZES = {
    # name: width, heads, key-value heads of the mixed-score attention, head size, rotated size, latent size, query latent size, dense ff,
    #       norm groups; Pomipel's experts, top, expert ff
    "w1024": (1024, 8, 2, 128, 64, 256, 512, 4096, 4, 16, 4, 512),
    "w2048": (2048, 16, 4, 128, 64, 512, 1024, 8192, 8, 32, 4, 1024),
    "w4096": (4096, 32, 8, 128, 64, 512, 1536, 14336, 8, 64, 6, 1024),
}


def run_fizadra_compare(args) -> None:
    from lit_gpt_b200 import kernels as K
    from lit_gpt_b200.config import (DenseMLPSpec, FizadraConfig, FizadraLayerSpec, LatentMixerSpec, LayerSpec, MoESpec, PomipelConfig, RotaryLatentSpec,
                                     RotarySpec, TalkingMixerSpec)
    from lit_gpt_b200.fizadra import Fizadra
    from lit_gpt_b200.latent import decode_splits
    from lit_gpt_b200.pomipel import Pomipel

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, peak_source = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    vocab, T = 32000, args.prompt
    iters = max(3, min(args.steps, 20))
    launches0 = K.launch_count()
    bf = torch.bfloat16
    out = {}
    for name in (args.sizes.split(",") if args.sizes else FIZADRA_SIZES):
        d, H, G, hs, dr, r, qr, dff, groups, E, top, ff = FIZADRA_SIZES[name]
        blended = RotarySpec(dims=dr, base=1e6, factor=4.0, original=4096.0, fast=32.0, slow=1.0)
        half = RotarySpec(dims=dr, base=1e6, interleaved=False)
        scale = (hs + dr) ** -0.5
        layers = [FizadraLayerSpec("latent_attention_2", RotaryLatentSpec(H, hs, dr, hs, r, qr, scale, half, gate="head"), DenseMLPSpec(dff)),
                  FizadraLayerSpec("latent_attention", RotaryLatentSpec(H, hs, dr, hs, r, qr, scale, blended, sink=True, gate="element"), DenseMLPSpec(dff)),
                  FizadraLayerSpec("attention", TalkingMixerSpec(H, G, hs, hs, hs ** -0.5, RotarySpec(dims=hs, base=1e6, interleaved=False)), DenseMLPSpec(dff)),
                  FizadraLayerSpec("latent_attention", RotaryLatentSpec(H, hs, dr, hs, r, qr, scale, blended, sink=True, gate="element", kv_from=1),
                                   DenseMLPSpec(dff))]
        fiz = Fizadra(FizadraConfig(vocab_size=vocab, n_embd=d, norm_groups=groups, layers=layers)).to(dev).to(bf).eval()
        fiz.reset_parameters()
        fiz.max_seq_length = T + 64
        players = [LayerSpec("latent_attention", LatentMixerSpec(H, hs, hs, r, qr, hs ** -0.5, None if i % 2 == 0 else i - 1),
                             MoESpec(E, top, ff, 4, 2)) for i in range(4)]
        pom = Pomipel(PomipelConfig(vocab_size=vocab, n_embd=d, block_size=T + 64, embedding_scale=d ** 0.5, logit_scale=1.0, layers=players))
        pom = pom.to(dev).to(bf).eval()
        pom.reset_parameters()
        res = {}
        with torch.inference_mode():
            for label, model in (("fizadra", fiz), ("pomipel", pom)):
                for B in (1, 8):
                    model.set_kv_cache(batch_size=B)
                    idx = torch.randint(0, vocab, (B, T), device=dev)
                    pos = torch.arange(T, device=dev)
                    if B == 1:
                        ms = _timed(lambda: model(idx, pos), iters, flush)
                        res[f"{label}_prefill_tok_s"] = round(T / ms * 1e3)
                    else:
                        model(idx, pos)
                    tok, p1 = idx[:, :1].contiguous(), torch.tensor([T], device=dev)
                    step, graphed = _graphed(lambda: model(tok, p1))
                    ms = _timed(step, iters, flush)
                    res[f"{label}_decode_b{B}_tok_s"] = round(B / ms * 1e3)
                    res[f"{label}_decode_b{B}_graphed"] = graphed
                    del step
                model.clear_kv_cache()
            kern = {}
            seqs = torch.tensor([[0, T, 0, 0]], dtype=torch.int32, device=dev)
            pairs = T * (T + 1) / 2
            # prompt attention over expanded keys and values: the rotated shared key part makes the query head hs + dr wide
            mx = fiz.blocks[1].mixer
            q = torch.randn(T, H * (hs + dr), device=dev, dtype=bf)
            kvp = torch.randn(T, 2 * H * hs, device=dev, dtype=bf)
            kr = torch.randn(T, dr, device=dev, dtype=bf)
            gate = torch.randn(T, H * hs, device=dev, dtype=bf)
            ms = _timed(lambda: K.latent_prefill(q, kvp[:, : H * hs], kvp[:, H * hs :], seqs, T, H, hs + dr, hs, scale, k_shared=kr, sink=mx.sink, gate=gate),
                        iters, flush)
            kern["prefill_latent_attention_fizadra"] = {"ms": ms, "frac_of_measured_bf16": 2.0 * H * (2 * hs + dr) * pairs / (ms * 1e-3) / tf}
            qp = torch.randn(T, H * hs, device=dev, dtype=bf)
            ms = _timed(lambda: K.latent_prefill(qp, kvp[:, : H * hs], kvp[:, H * hs :], seqs, T, H, hs, hs, hs ** -0.5), iters, flush)
            kern["prefill_attention_pomipel"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * H * hs * pairs / (ms * 1e-3) / tf}
            # prompt attention with mixed scores, over the cache rows
            ta = fiz.blocks[2].mixer
            kc, vc = torch.randn(T, G * hs, device=dev, dtype=bf), torch.randn(T, G * hs, device=dev, dtype=bf)
            ms = _timed(lambda: K.talk_attn(qp, kc, vc, seqs, T, H, G, hs, hs, T, hs ** -0.5, 1, talk=ta.talk, sink=ta.sink, context=T), iters, flush)
            kern["prefill_mixed_score_attention_fizadra"] = {"ms": ms, "frac_of_measured_bf16": (4.0 * H * hs + 2.0 * H * H) * pairs / (ms * 1e-3) / tf,
                                                             "plane_bytes_moved": 4.0 * H * pairs * 4, "frac_of_measured_hbm_for_planes": 4.0 * H * pairs * 4 / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.talk_attn(qp, kc, vc, seqs, T, H, G, hs, hs, T, hs ** -0.5, 1, talk=ta.talk, sink=ta.sink), max(2, iters // 4), flush)
            kern["prefill_mixed_score_attention_any_size_kernel_fizadra"] = {"ms": ms, "fp32_tflops": (4.0 * H * hs + 2.0 * H * H) * pairs / (ms * 1e-3) / 1e12}
            # single rows
            B = 8
            slot = torch.arange(B, dtype=torch.int32, device=dev)
            rp = torch.full((B,), T - 1, dtype=torch.int32, device=dev)
            qd = torch.randn(B, H * (hs + dr), device=dev, dtype=bf)
            cache = torch.randn(B, T, r + dr, device=dev, dtype=bf)
            gd = torch.randn(B, H * hs, device=dev, dtype=bf)
            tiles = -(-H // 16)
            ms = _timed(lambda: K.latent_decode(qd, mx.w_uk, mx.w_uv, cache, slot, rp, H, hs, hs, scale, decode_splits(T, B * tiles), shared_dims=dr,
                                                sink=mx.sink, gate=gd), iters, flush)
            roof = max(B * T * (r + dr) * 2 / hbm, 2.0 * B * H * T * (2 * r + dr) / tf)
            kern["decode_latent_attention_fizadra"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": B * T * (r + dr) * 2}
            pm = pom.blocks[0].mixer
            qdp, cp = torch.randn(B, H * hs, device=dev, dtype=bf), torch.randn(B, T, r, device=dev, dtype=bf)
            ms = _timed(lambda: K.latent_decode(qdp, pm.w_uk, pm.w_uv, cp, slot, rp, H, hs, hs, hs ** -0.5, decode_splits(T, B * tiles)), iters, flush)
            roof = max(B * T * r * 2 / hbm, 4.0 * B * H * T * r / tf)
            kern["decode_attention_pomipel"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": B * T * r * 2}
            kcb, vcb = torch.randn(B * T, G * hs, device=dev, dtype=bf), torch.randn(B * T, G * hs, device=dev, dtype=bf)
            sq1 = torch.tensor([(b, 1, T - 1, b) for b in range(B)], dtype=torch.int32, device=dev)
            ms = _timed(lambda: K.talk_attn(qdp, kcb, vcb, sq1, 1, H, G, hs, hs, T, hs ** -0.5, decode_splits(T, B), talk=ta.talk, sink=ta.sink), iters, flush)
            roof = 2.0 * B * T * G * hs * 2 / hbm
            kern["decode_mixed_score_attention_fizadra"] = {"ms": ms, "roofline_ms": roof * 1e3, "frac_of_roofline": roof / (ms * 1e-3), "bytes": 2.0 * B * T * G * hs * 2}
            # residual kernels: post-norm in groups + sum + sum over five results + next pre-norm, against Pomipel's norm + sum
            x = torch.randn(T, d, device=dev, dtype=bf)
            stack = torch.randn(5, T, d, device=dev)
            xs, avg, act = torch.randn(T, d, device=dev), torch.empty(T, d, device=dev), torch.empty(T, d, device=dev, dtype=bf)
            blk = fiz.blocks[3]
            ms = _timed(lambda: K.depth_residual(xs, stack[4], 1e-5, groups, y=x, post_w=blk.norm_2b, stack=stack, m=5, depth_w=blk.dwa, avg=avg,
                                                 pre_w=blk.norm_1, act=act), iters, flush)
            kern["residual_with_depth_sum_fizadra"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 4 + 4 + 4 * 4 + 4 + 2) / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.depth_residual(xs, xs, 1e-5, groups, y=x, post_w=blk.norm_1b, pre_w=blk.norm_2, act=act), iters, flush)
            kern["residual_fizadra"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            ms = _timed(lambda: K.residual_norm_add(x, pom.blocks[0].norm_1, 1e-5, xs, act), iters, flush)
            kern["residual_norm_pomipel"] = {"ms": ms, "frac_of_measured_hbm": T * d * (2 + 4 + 4 + 2) / (ms * 1e-3) / hbm}
            # per-head norm + rotation + cache store of a fused q | k | v projection, beside Pomipel's norm of projected rows
            cols = (H + 2 * G) * hs
            qkv = torch.randn(T, cols, device=dev, dtype=bf)
            kcache, vcache = torch.empty(T, G * hs, device=dev, dtype=bf), torch.empty(T, G * hs, device=dev, dtype=bf)
            rows64, pos32 = torch.arange(T, device=dev), torch.arange(T, device=dev, dtype=torch.int32)
            fr = ta.freq(dev)
            segs = [K.rope_seg(qkv[:, : H * hs], qkv[:, : H * hs], H, hs, norm_w=ta.q_norm, freq=fr, rot_dims=hs, interleaved=False),
                    K.rope_seg(qkv[:, H * hs : (H + G) * hs], kcache, G, hs, norm_w=ta.k_norm, freq=fr, rot_dims=hs, interleaved=False, out_rows=rows64),
                    K.rope_seg(qkv[:, (H + G) * hs :], vcache, G, hs, out_rows=rows64)]
            ms = _timed(lambda: K.head_rope(T, pos32, 1e-5, *segs, dtype=bf, device=dev), iters, flush)
            kern["head_norm_rotation_store_fizadra"] = {"ms": ms, "frac_of_measured_hbm": T * cols * 4.0 / (ms * 1e-3) / hbm}
            down, cq = torch.randn(T, cols, device=dev, dtype=bf), torch.empty(T, cols, device=dev, dtype=bf)
            wn = torch.ones(cols, device=dev, dtype=bf)
            ms = _timed(lambda: K.rms_rows(T, 1e-5, K.rms_seg(down, wn, cq, cols, False), in_dtype=bf, out_dtype=bf, device=dev), iters, flush)
            kern["norm_of_projected_rows_pomipel"] = {"ms": ms, "frac_of_measured_hbm": T * cols * 4.0 / (ms * 1e-3) / hbm}
            ms = _timed(lambda: fiz.blocks[0].mlp(x), iters, flush)
            kern["dense_mlp_fizadra"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * T * dff * d / (ms * 1e-3) / tf}
            ms = _timed(lambda: pom.blocks[0].mlp(x), iters, flush)
            kern["experts_pomipel"] = {"ms": ms, "frac_of_measured_bf16": 4.0 * T * top * ff * d / (ms * 1e-3) / tf}
            res["kernels"] = {k: {a: (round(b, 4) if isinstance(b, float) else b) for a, b in v.items()} for k, v in kern.items()}
        out[name] = res
        del fiz, pom
        torch.cuda.empty_cache()
    print(json.dumps({"compare": "fizadra", "layers": 4, "prompt": T, "context": T, "dtype": "bf16", "data": "synthetic, random weights",
                      "l2": "flushed between timed calls", "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                                                                       "source": peak_source},
                      "gpu_launches": int(K.launch_count() - launches0), "sizes": out}), flush=True)


def main() -> None:
    # stdout carries exactly one JSON line: NCCL's own banner / debug lines (when the box sets NCCL_DEBUG) go to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":  # the version banner is printf'd to stdout whatever the file is
        os.environ["NCCL_DEBUG"] = "WARN"
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="llama2-7b-nf4-bs1")
    ap.add_argument("--layers", type=int, default=None, help="debug only: build fewer blocks (invalidates the number)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--compare", choices=["pomipel", "lefalix", "fizadra", "nulezen"], default=None,
                    help="instead of the default workload: prefill / decode throughput of that design beside the closest existing model")
    ap.add_argument("--sizes", default=None, help=f"--compare: comma-separated subset of {sorted(ARCH_SIZES)} (the same names for both designs)")
    ap.add_argument("--prompt", type=int, default=2048, help="--compare: prompt and context length")
    args = ap.parse_args()
    if args.compare == "nulezen":
        run_nulezen_compare(args)
        return
    if args.compare == "fizadra":
        run_fizadra_compare(args)
        return
    if args.compare == "lefalix":
        run_lefalix_compare(args)
        return
    if args.compare:
        run_arch_compare(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        teardown()


def teardown() -> None:
    """Orderly multi-rank exit: captured graphs and peer mappings are dropped BEFORE the process group (a CUDA graph that
    captured an NCCL collective keeps the communicator busy: destroying the group first is what used to hang).  A watchdog
    turns a teardown that still does not finish within 30 s into a plain exit, after everything has been printed."""
    import gc

    import torch.distributed as dist

    sys.stdout.flush()
    sys.stderr.flush()

    def _bail():
        sys.stderr.write("bench.py: teardown did not finish within 30 s; leaving without destructors\n")
        sys.stderr.flush()
        os._exit(0)

    wd = threading.Timer(30.0, _bail)
    wd.daemon = True
    wd.start()
    torch.cuda.synchronize()
    dist.barrier()
    for obj in gc.get_objects():
        try:
            if type(obj).__name__ == "GPT" and hasattr(obj, "__dict__"):
                obj.__dict__.pop("_decode_graphs", None)
                comm = obj.__dict__.pop("_p2p", None)
                if comm:
                    comm.close()
        except Exception:
            pass
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    wd.cancel()


if __name__ == "__main__":
    main()
