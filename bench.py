"""Prefill throughput of the Qwen3.5-style hybrid decoder on B200, one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (every N): the 4B-shaped decoder of BASELINE.json's second config - 32 layers, three
Gated DeltaNet to one gated GQA attention layer, hidden 2560, MLP 9728, vocab 151936, bf16
weights N(0, 0.02) generated on the device - prefilling one request of 1024 uniform-random
token ids per GPU (weak scaling: requests shard across GPUs with replicated weights; the
only exchange is the gather of the 16 decision logits to rank 0). A step is one prefill.

One JSON line on rank 0:
  value      tokens/s over all GPUs with the ids already in HBM, device-timed (CUDA events on
             the executor's stream, max over ranks)
  e2e        the same through the public call with host buffers: pinned ids -> H2D -> layers ->
             last row D2H -> float64 head on the host (-> NCCL gather of logits when N > 1)
  roofline   the dominant kernel family (the bf16 GEMMs): algorithmic FLOPs per step over its
             device time, measured with events around every launch in profiled steps
  cpu_baseline  the CPU oracle (a port of the reference's arithmetic, OpenMP) on a bounded
             sample of the same workload, N = 1 only
--impl reference times that CPU oracle as the reference arm (the reference has no CPU
forward pass of its own: its CPU code for this path is the float64 test oracles the port restates).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOKENS = 1024
N_CLASSES = 16
WORKLOAD = ("cfg2: 4B-shaped hybrid decoder (32 layers 3:1 GDN/attention, hidden 2560, MLP 9728, vocab 151936, "
            "16-class head), 1 request x 1024 uniform-random ids per GPU")
# DRAM bytes of one launch of the pair kernel (ncu, dram__bytes_read.sum + dram__bytes_write.sum) on the
# widest projection of this workload; the capture and its command are under profiles/.
GEMM_TRAFFIC = {"bytes": 72.9e6,
                "of": "one launch, y[1024,12352] = x[1024,2560] w^T (GDN in_proj): algorithmic 93.7e6 bytes "
                      "(x 5.2e6 + w 63.2e6 + y 25.3e6, most of y still in L2 when the launch ends)"}
FAMILIES = ["gemm", "gdn_prefill", "attention", "gdn_conv", "gdn_gates", "rms_norm", "gated_rms_norm", "silu_mul",
            "attn_prep", "other"]


def cfg2(layers=32):
    from system1_omni_b200.model import Config
    types = [("full_attention" if (i + 1) % 4 == 0 else "linear_attention") for i in range(layers)]
    return Config(hidden=2560, intermediate=9728, layer_types=types, heads=16, kv_heads=4, head_dim=128,
                  rotary_half=32, lin_k_heads=16, lin_v_heads=32, vocab=151936, eps=1e-6, rope_theta=1e7,
                  max_positions=262144)


def gemm_flops_per_token(cfg):
    """2*N*K summed over the projections of every layer: the GEMM FLOPs one token costs."""
    h, I, kd, vd, hv = cfg.hidden, cfg.intermediate, cfg.key_dim, cfg.value_dim, cfg.lin_v_heads
    gdn = (2 * kd + vd + vd + 2 * hv) * h + h * vd
    att = (cfg.heads * cfg.head_dim * 2 + 2 * cfg.kv_heads * cfg.head_dim) * h + h * cfg.heads * cfg.head_dim
    mlp = 2 * I * h + h * I
    total = 0
    for full in cfg.full_attention:
        total += (att if full else gdn) + mlp
    return 2 * total


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"tflops": p.get("bf16_tflops_sustained", 1389.8), "hbm_gbs": p.get("hbm_gbs", 6543.7),
                "source": "measured"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while running."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.lines = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def cpu_sample(periods=1, seed=0):
    """The CPU oracle on `periods` x (3 Gated DeltaNet + 1 attention) layers of the workload's
    shape at 1024 tokens, random hidden states in. Returns (seconds, layers run, threads)."""
    import oracle as O
    cfg = cfg2(4 * periods)
    from system1_omni_b200.model import tensor_shapes
    rng = np.random.default_rng(seed)
    cache, weights = {}, {}
    for name, shape in tensor_shapes(cfg).items():
        if name == "embed_tokens.weight":
            weights[name] = np.zeros((1, cfg.hidden), np.uint16)      # not read: hidden states are given
            continue
        # layers of every period share one set of arrays: the arithmetic and its cost are the same
        parts = name.split(".")
        key = ".".join([str(int(parts[1]) % 4)] + parts[2:]) if parts[0] == "layers" else name
        if key not in cache:
            n = int(np.prod(shape))
            if name.endswith("A_log"):
                a = rng.uniform(0, np.log(16), n).astype(np.float32)
            elif name.endswith("dt_bias"):
                a = rng.normal(0, 0.1, n).astype(np.float32)
            elif name.endswith("linear_attn.norm.weight"):
                a = (1 + rng.normal(0, 0.02, n)).astype(np.float32)
            else:
                a = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
            cache[key] = O.f32_to_bf16(a).reshape(shape)
        weights[name] = cache[key]
    x = O.f32_to_bf16(rng.standard_normal((TOKENS, cfg.hidden), dtype=np.float32))
    d = cfg.oracle_dict()
    d["vocab"] = 1
    t0 = time.perf_counter()
    O.forward(d, weights, None, [TOKENS], x_in=x)
    return time.perf_counter() - t0, cfg.n_layers, O.threads()


def run_reference(args, rank, world):
    """The reference arm: the reference project has no CPU forward pass, so its arithmetic as
    restated by the oracle is timed on the host cores; each step is one period (4 layers) of
    the 32-layer workload at 1024 tokens, scaled by 32/4."""
    if rank != 0:
        return
    secs = []
    layers = threads = None
    for i in range(args.warmup + args.steps):
        if i >= 1 and sum(secs) > 240:       # keep the whole run within a few minutes
            break
        t, layers, threads = cpu_sample(1, seed=i)
        if i >= min(args.warmup, 1):
            secs.append(t)
    step = float(np.mean(secs)) * 32 / layers
    value = TOKENS / step
    sample = (f"oracle port, {layers} of 32 layers (one 3 GDN + 1 attention period) at {TOKENS} tokens, "
              f"time x {32 // layers}, {len(secs)} timed samples")
    line = {"impl": "reference", "metric": "prefill tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(secs), "warmup": min(args.warmup, 1), "ms_per_step": step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers": 32, "tokens_per_gpu": TOKENS,
                       "weights": "N(0,0.02) bf16, generated on the host"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=32, help="fewer layers for a quick functional check only")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graphs", type=int, default=1, help="CUDA-graph replay of the layer loop (0 = eager)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    dist = torch = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        # Whatever NCCL prints while its communicator comes up (a version banner, when the environment
        # asks for one) goes to stderr: stdout carries the one JSON line.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    from system1_omni_b200 import lib as L
    from system1_omni_b200 import model as M
    lib = L.load()                  # raises when the CUDA library is missing: there is no other path
    L.set_device(local)
    cfg = cfg2(args.layers)
    model = M.Model(cfg, device=local)
    model.init_random(seed=0, std=0.02)
    stream = model.stream
    rng = np.random.default_rng(1000 + rank)
    ids = rng.integers(0, cfg.vocab, TOKENS).astype(np.int32)
    head = np.random.default_rng(7).normal(0, 1.0, (N_CLASSES, cfg.hidden)).astype(np.float32)
    lengths = np.array([TOKENS], np.int32)

    # pinned host ids for the end-to-end leg, device-resident ids for the kernel leg
    pinned = C.c_void_p()
    L.check(lib.s1_host_alloc(C.byref(pinned), ids.nbytes), "pinned")
    host_ids = np.ctypeslib.as_array(C.cast(pinned, C.POINTER(C.c_int32)), shape=(TOKENS,))
    host_ids[:] = ids
    ids_dev = L.DeviceBuffer(ids.nbytes)
    L.check(lib.cs1_upload(ids_dev.at(), pinned, ids.nbytes, stream), "upload ids")

    def barrier():
        model.synchronize()
        if dist:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if not dist:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    model.enable_graphs(bool(args.graphs))
    for _ in range(args.warmup):
        model.forward_device(ids_dev.at(), lengths)
    model.synchronize()
    lib.s1_model_profile_read(model.handle, None, None, None)      # reset the launch counters

    sampler = ClockSampler(local)
    # ---- device-timed steps, ids resident in HBM ----
    e0, e1 = L.Event(), L.Event()
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        model.forward_device(ids_dev.at(), lengths)
    e1.record(stream)
    barrier()
    ms_total = max_over_ranks(e0.elapsed_ms(e1))
    launches = (C.c_longlong * len(FAMILIES))()
    lib_launches = C.c_longlong()
    L.check(lib.s1_model_profile_read(model.handle, None, launches, C.byref(lib_launches)), "profile read")
    stats = model.graph_stats()
    ms_step = ms_total / args.steps
    value = world * TOKENS / (ms_step * 1e-3)

    # ---- end to end through the public call, host buffers ----
    logits_all = None
    gather_buf = [torch.zeros(N_CLASSES, device="cuda") for _ in range(world)] if dist else None

    def e2e_step():
        last = model.forward_flat(host_ids, lengths)
        logits = M.head_logits(head, last[0])
        if dist:
            dist.all_gather(gather_buf, torch.from_numpy(logits).cuda())
            return torch.stack(gather_buf).cpu().numpy()
        return logits[None]

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        logits_all = e2e_step()
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / args.steps
    clocks = sampler.stop()
    decisions = [int(M.answer(row)[0]) for row in logits_all]

    # ---- per-family device time: eager profiled steps right after the timed ones ----
    model.enable_graphs(False)
    lib.s1_model_profile(model.handle, 1)
    prof_steps = 3
    for _ in range(prof_steps):
        model.forward_device(ids_dev.at(), lengths)
    fam_ms = (C.c_float * len(FAMILIES))()
    fam_launch = (C.c_longlong * len(FAMILIES))()
    fam_lib = C.c_longlong()
    L.check(lib.s1_model_profile_read(model.handle, fam_ms, fam_launch, C.byref(fam_lib)), "profile read")
    lib.s1_model_profile(model.handle, 0)
    per_family = {name: {"ms_per_step": fam_ms[i] / prof_steps, "launches_per_step": fam_launch[i] / prof_steps}
                  for i, name in enumerate(FAMILIES)}
    gemm_ms = per_family["gemm"]["ms_per_step"]
    gemm_launches = (fam_launch[0] + fam_lib.value) / prof_steps
    flops = gemm_flops_per_token(cfg) * TOKENS
    pk = peaks()
    achieved = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    engine = "tcgen05 (this library)" if fam_launch[0] > 0 else "cuBLASLt"

    if rank != 0:
        model.close()
        if dist:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        secs, layers, threads = cpu_sample(1)
        cpu = {"value": TOKENS / (secs * cfg.n_layers / layers), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"oracle port on {layers} of {cfg.n_layers} layers (one 3 GDN + 1 attention period) at "
                         f"{TOKENS} tokens, {secs:.1f} s, scaled by {cfg.n_layers}/{layers}"}
    own_per_step = int(sum(fam_launch)) // prof_steps
    own = int(sum(launches)) + int(stats["replays"]) * own_per_step      # a replay launches a whole step's kernels
    line = {
        "metric": "prefill tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": cfg.n_layers, "tokens_per_gpu": TOKENS, "weights": "N(0,0.02) bf16, generated on device",
                   "l2": f"per step {model.weight_bytes / 1e9:.1f} GB of weights stream through a 126 MB L2",
                   "graphs": bool(args.graphs), "gemm_engine": engine},
        "e2e": {"value": world * TOKENS / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(ids.nbytes + 4), "d2h_bytes_per_step": int(cfg.hidden * 2)},
        "gpu_launches": own,
        "launch_detail": {"own_kernels_in_timed_region": own,
                          "own_kernels_launched_eagerly_in_timed_region": int(sum(launches)), "library_launches_in_timed_region": int(lib_launches.value),
                          "graph_replays": stats["replays"], "own_kernels_per_eager_step": own_per_step,
                          "library_launches_per_eager_step": int(fam_lib.value) // prof_steps},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                     "frac": achieved / pk["tflops"], "traffic": GEMM_TRAFFIC["bytes"] if fam_launch[0] > 0 else None,
                     "traffic_of": GEMM_TRAFFIC["of"], "kernel": f"bf16 GEMM, {engine}",
                     "launches_per_step": gemm_launches, "flops_per_step": flops, "ms_per_step": gemm_ms,
                     "peak_source": pk["source"] + " (sustained cuBLAS bf16)"},
        "per_family": per_family,
        "clocks": clocks,
        "decisions": decisions,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    model.close()
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
