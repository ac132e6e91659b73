"""Benchmark of the dnn.c training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE config 5): one training step (forward, backward, gradient
clipping, AdamW, cosine LR) of the GPT-124M-shaped decoder LM -- vocab 32000,
d_model 768, 12 blocks, 12 heads x 64, SwiGLU hidden 2048, RoPE, RMSNorm, tied
head, fp32 parameters and optimiser state -- on a micro-batch of 16 x 1024
synthetic tokens per GPU, called through the C-ABI of libdnn_b200.so.
Metric: training tokens per second, whole job.  N > 1 is data parallel (one
process per GPU, launched by torchrun), gradients averaged over NCCL.

`--impl reference` times the reference's own CPU implementation (oracle/_ref,
built from the reference sources by oracle/Makefile) on a bounded sample of the
same workload on the host cores.
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
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

CFG = dict(V=32000, D=768, L=12, H=12, F=2048, B=16, N=1024, lr=6e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, clip=1.0,
           warmup_iters=100, total_iters=10000, seed=4)
# the bounded CPU sample: the full 12-block model and code path on one short sequence
CPU_SAMPLE = dict(CFG, B=1, N=16)
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libdnn_ref.so")
METRIC = "train tokens/s (fwd+bwd+AdamW), 12L-768d GPT"
# DRAM bytes (read + write) the GEMM kernel moves per training step of CFG in TF32 mode, from an
# ncu capture of every linear-layer shape at full size, forward, dA and dW (summary:
# profiles/gemm_tf32_kernel_linear_shapes.txt): 2.603 GB per transformer block; the three launches
# of the vocabulary projection (6.7 GB working set, not captured) are taken at their algorithmic
# bytes.  183 GEMM launches per step; `roofline.traffic` is the per-launch average.
GEMM_DRAM_BYTES_PER_STEP = 12 * 2.603e9 + 6.73e9
GEMM_LAUNCHES_PER_STEP = 183


def param_names(L):
    names = ["embed.weight"]
    for i in range(L):
        p = "blocks.%d." % i
        names += [p + s for s in ("qkv_proj.weight", "qkv_proj.bias", "out_proj.weight", "out_proj.bias", "attn_norm.weight",
                                  "ffn_norm.weight", "ffn.gate_proj.weight", "ffn.gate_proj.bias", "ffn.up_proj.weight",
                                  "ffn.up_proj.bias", "ffn.down_proj.weight", "ffn.down_proj.bias")]
    return names + ["norm.weight", "lm_head.bias"]


def build_model(dnn, B, cfg):
    """decoder_lm + AdamW + LR scheduler through the C API; N(0, 0.02) weights from a fixed seed."""
    lib = dnn.lib
    lm = lib.decoder_lm_create(dnn.params, cfg["V"], cfg["D"], cfg["L"], cfg["H"], cfg["D"] // cfg["H"], cfg["F"])
    lib.decoder_lm_enable_rope(dnn.params, lm, cfg["N"], 10000.0)
    params = dnn.parameters(lm)
    rng = np.random.default_rng(cfg["seed"])
    for t, name in zip(params, param_names(cfg["L"])):
        shape = dnn.shape_of(t)
        if name.endswith("norm.weight"):
            v = np.ones(shape, np.float32)
        elif name.endswith("bias"):
            v = np.zeros(shape, np.float32)
        else:
            v = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
        dnn.upload(t, v)
    arr = (B.TensorP * len(params))(*params)
    opt = lib.adamw_create(dnn.params, arr, len(params), cfg["lr"], cfg["b1"], cfg["b2"], cfg["eps"], cfg["wd"])
    sched = lib.lr_scheduler_create(dnn.params, opt, 1, cfg["lr"], cfg["warmup_iters"], cfg["total_iters"], -1.0, 0, 0.0)
    return lm, opt, sched, params, arr


def token_batch(cfg, rank, step):
    rng = np.random.default_rng([cfg["seed"] + rank, step])
    return rng.integers(0, cfg["V"], size=(cfg["B"], cfg["N"]), dtype=np.int32)


class ClockSampler:
    """nvidia-smi SM clock and throttle reasons, sampled every 200 ms while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["bf16_tflops_sustained"], p["hbm_gbs"], "measured"
    return 1400.0, 6650.0, "fallback"


def run_cpu_sample(B, steps, warmup, threads):
    """Reference CPU implementation on the bounded sample; returns (tokens/s, s/step)."""
    os.environ["OMP_NUM_THREADS"] = str(threads)
    ref = B.Dnn(REF_LIB, params_mb=4096, scratch_mb=8192, data_mb=64)
    cfg = CPU_SAMPLE
    lm, opt, sched, params, arr = build_model(ref, B, cfg)
    times = []
    for s in range(warmup + steps):
        ids_np = token_batch(cfg, 0, s)
        t0 = time.perf_counter()
        ids = ref.tensor(ids_np, ref.data)
        tgt = ref.lib.decoder_lm_shift_targets(ref.data, ids)
        gn = C.c_float(0)
        loss = ref.lib.decoder_lm_train_step(ref.scratch, lm, ids, tgt, opt, cfg["clip"], C.byref(gn))
        ref.lib.lr_scheduler_step(sched)
        _ = ref.scalar(loss)
        dt = time.perf_counter() - t0
        ref.reset_step()
        if s >= warmup:
            times.append(dt)
    ref.close()
    sec = float(np.mean(times))
    return cfg["B"] * cfg["N"] / sec, sec


def cpu_baseline_obj(value, threads):
    return {"value": round(value, 2), "unit": "tokens/s", "cores": threads, "kind": "reference",
            "sample": "full 12-block model, one training step on a batch of %d x %d tokens instead of 16 x 1024 (NO_CBLAS, non-NEON "
                      "build of the reference, %d OpenMP threads)" % (CPU_SAMPLE["B"], CPU_SAMPLE["N"], threads)}


def reference_arm(args, B, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    if not os.path.exists(REF_LIB):
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libdnn_ref.so is not built on this machine"}))
        return
    steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
    tps, sec = run_cpu_sample(B, steps, warmup, threads)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(tps, 2), "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gpt124m-shaped decoder LM train step (BASELINE config 5), bounded sample: batch 1 x 16 tokens"},
        "cpu_baseline": cpu_baseline_obj(tps, threads),
        "e2e": {"value": round(tps, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--gemm", default="tf32", choices=["tf32", "3xtf32", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    B = entry.load_binding()
    if args.impl == "reference":
        reference_arm(args, B, rank)
        return
    assert args.warmup >= 3, "timing rules: at least 3 warm-up steps"
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    cfg = CFG
    dnn = B.Dnn(B.B200_LIB, params_mb=3072, scratch_mb=56 * 1024, data_mb=64, device=local)
    lib = dnn.lib
    lib.dnn_cuda_set_gemm_mode({"fp32": 0, "tf32": 1, "3xtf32": 2}[args.gemm])
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = (C.c_ubyte * 128)()
            assert lib.dnn_cuda_dp_unique_id(buf) == 0
            idt.copy_(torch.tensor(list(buf), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        idb = (C.c_ubyte * 128)(*idt.cpu().tolist())
        assert lib.dnn_cuda_dp_init(rank, world, idb) == 0, "dnn_cuda_dp_init failed"
    lm, opt, sched, params, arr = build_model(dnn, B, cfg)
    n_params = sum(int(np.prod(dnn.shape_of(t))) for t in params)
    tokens = cfg["B"] * cfg["N"]
    step_fn = lib.dnn_cuda_dp_decoder_lm_train_step

    pinned = lib.dnn_cuda_host_alloc(tokens * 4)
    pinned_np = np.ctypeslib.as_array(C.cast(pinned, C.POINTER(C.c_int32)), shape=(cfg["B"], cfg["N"]))
    loss_host = np.zeros(1, np.float32)

    def one_step(step, resident_ids=None):
        """One training step.  resident_ids: device tensor already holding the batch (kernel-timed
        loop) or None (end-to-end loop: the batch comes from pinned host memory)."""
        if resident_ids is None:
            ids = lib.tensor_scratch(dnn.data, 2, B.ints([cfg["B"], cfg["N"]]), 0)
            lib.dnn_cuda_upload(ids, pinned, tokens * 4)
        else:
            ids = resident_ids
        tgt = lib.decoder_lm_shift_targets(dnn.data, ids)
        gn = C.c_float(0)
        loss = step_fn(dnn.scratch, lm, ids, tgt, opt, cfg["clip"], C.byref(gn))
        lib.lr_scheduler_step(sched)
        return loss, gn.value

    def barrier():
        lib.dnn_cuda_sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # batches for the kernel-timed loop are resident before the clock starts
    total = args.warmup + args.steps
    resident = dnn.tensor(token_batch(cfg, rank, 0), dnn.params)     # params pool: survives reset_step

    for s in range(args.warmup):
        loss, gn = one_step(s, resident)
        lib.dnn_cuda_sync()
        dnn.lib.dnn_ctx_reset_step(C.byref(dnn.ctx))

    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = lib.dnn_cuda_launch_count()
    lib.dnn_cuda_profile_enable(1)
    lib.dnn_cuda_timer_start()
    losses = []
    for s in range(args.steps):
        loss, gn = one_step(args.warmup + s, resident)
        dnn.lib.dnn_ctx_reset_step(C.byref(dnn.ctx))        # bump pointers only; stream order keeps reuse safe
    ms_total = lib.dnn_cuda_timer_stop_ms()
    barrier()
    launches = lib.dnn_cuda_launch_count() - launches0
    nl, gms, gwork = C.c_longlong(0), C.c_double(0), C.c_double(0)
    lib.dnn_cuda_profile_read(0, C.byref(nl), C.byref(gms), C.byref(gwork))
    al, ams, awork = C.c_longlong(0), C.c_double(0), C.c_double(0)
    lib.dnn_cuda_profile_read(1, C.byref(al), C.byref(ams), C.byref(awork))
    lib.dnn_cuda_profile_enable(0)
    clocks = sampler.stop() if rank == 0 else None

    # end-to-end: batch from pinned host memory every step, loss read back every step
    barrier()
    t_e2e0 = time.perf_counter()
    lib.dnn_cuda_timer_start()
    for s in range(args.steps):
        pinned_np[...] = token_batch(cfg, rank, total + s)
        loss, gn = one_step(total + s, None)
        lib.dnn_cuda_download(loss, loss_host.ctypes.data, 4)
        losses.append(float(loss_host[0]))
        dnn.lib.dnn_ctx_reset_step(C.byref(dnn.ctx))
    ms_e2e_dev = lib.dnn_cuda_timer_stop_ms()
    ms_e2e = max(ms_e2e_dev, (time.perf_counter() - t_e2e0) * 1e3)

    if dist is not None:
        t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e = float(t[0]), float(t[1])
    ms_step = ms_total / args.steps
    value = world * tokens / (ms_step / 1e3)
    e2e_value = world * tokens / (ms_e2e / args.steps / 1e3)

    if rank == 0:
        bf16_sustained, hbm, src = peaks()
        tf32_peak = 0.5 * bf16_sustained
        achieved = gwork.value / (gms.value * 1e-3) / 1e12 if gms.value > 0 else 0.0
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"tf32": "tf32", "3xtf32": "3xtf32", "fp32": "f32"}[args.gemm], "data": "synthetic",
            "config": {"workload": "gpt124m-shaped decoder LM train step (BASELINE config 5)", "vocab": cfg["V"], "d_model": cfg["D"],
                       "n_layers": cfg["L"], "n_heads": cfg["H"], "ffn_hidden": cfg["F"], "micro_batch_per_gpu": cfg["B"],
                       "seq_len": cfg["N"], "global_batch_tokens": world * tokens, "params": n_params,
                       "parallelism": "dp%d" % world, "l2_flush": "inputs larger than L2 (activations ~30 GB per step)"},
            "roofline": {"bound": "tensor", "kernel": "gemm_tf32_kernel", "achieved": round(achieved, 1), "peak": round(tf32_peak, 1),
                         "unit": "TFLOP/s", "frac": round(achieved / tf32_peak, 4),
                         "traffic": round(GEMM_DRAM_BYTES_PER_STEP / GEMM_LAUNCHES_PER_STEP) if args.gemm == "tf32" and cfg == CFG else None,
                         "traffic_unit": "bytes per launch (DRAM read + write, ncu)",
                         "launches": nl.value, "kernel_ms_per_step": round(gms.value / args.steps, 3),
                         "flop_per_step": gwork.value / args.steps,
                         "peak_source": "0.5 x bf16_tflops_sustained of MEASURED_PEAKS.json (%s); no TF32 figure is measured there" % src,
                         "adamw": {"bound": "hbm", "achieved": round(awork.value / (ams.value * 1e-3) / 1e9, 1) if ams.value > 0 else None,
                                   "peak": hbm, "unit": "GB/s",
                                   "frac": round(awork.value / (ams.value * 1e-3) / 1e9 / hbm, 4) if ams.value > 0 else None}},
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": tokens * 4, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "clocks": clocks, "loss_first_last": [losses[0], losses[-1]] if losses else None,
            "scratch_peak_gb": round(lib.dnn_cuda_pool_device_peak(dnn.scratch) / 2 ** 30, 2),
        }
        if not args.no_cpu_baseline and world == 1 and os.path.exists(REF_LIB):
            threads = os.cpu_count() or 1
            tps, _ = run_cpu_sample(B, 1, 0, threads)
            out["cpu_baseline"] = cpu_baseline_obj(tps, threads)
        elif world == 1:
            out["cpu_baseline"] = None
        print(json.dumps(out))
    lib.dnn_cuda_host_free(pinned)
    if world > 1:
        lib.dnn_cuda_dp_finalize()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
