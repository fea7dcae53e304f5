#!/usr/bin/env python
"""Benchmark of the device path on the BASELINE configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step = one Execute of one loaded VMProgram (one megakernel launch; config 3 on N > 1
GPUs: gradient program, NCCL all-reduce, SGD program) on synthetic inputs of the
configuration's shapes and distributions (seeded; see pjrt-ocl_b200/programs/cases.py).
The default workload is the headline metric: config 5's pre-norm transformer block,
tokens/s, batch-sharded over the GPUs. `value` is measured with the arguments already
resident in HBM (CUDA events on the launching stream); `e2e` goes through the
host-buffer Execute call (pinned host -> device, launch, device -> host every step).
After the timed loop one step's results are copied back and checked by value
(tests/fullsize_refs.py): the line carries `"verified": true|false`.

`--impl reference` times the CPU arm: the reference's device kernels are OpenCL C and
cannot be built or run on this box, so the arm is the C restatement of the reference's
per-phase host walk and CPU tile bodies (oracle/), on all host cores, one bounded
sample of the workload per step (the sample is named in the line's `config`).
"""
from __future__ import annotations

import argparse
import gzip
import importlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PROG_DIR = os.path.join(ROOT, "pjrt-ocl_b200", "programs")
for p in (ROOT, PROG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

import inputs as gen_inputs  # noqa: E402

N_C2 = 8192 * 4096

# name -> program blob, CPU-arm sample blob (+ fraction of the full workload it is),
# algorithmic bytes per step, metric
def _wl(program, metric, unit, alg, scale, bound, dtype, desc, roof_alg=None, sample=None, sample_frac=0.0,
        secondary=False, plan=None, traffic=None, max_steps=None, sample_what=""):
    """alg: algorithmic units one step processes (bytes, flops or tokens); value = alg / seconds / scale.
    roof_alg: bytes (bound "hbm") or flops (bound "tensor") of one step, for the roofline fraction.
    traffic: dram__bytes_read.sum + dram__bytes_write.sum of one launch from the ncu capture summarised under
    profiles/ (bytes), where one was taken. max_steps: cap on timed steps where one step runs for a second or so."""
    return dict(program=program, metric=metric, unit=unit, alg=alg, scale=scale, bound=bound, dtype=dtype, desc=desc,
                roof_alg=alg if roof_alg is None else roof_alg, sample=sample, sample_frac=sample_frac,
                secondary=secondary, plan=plan, traffic=traffic, max_steps=max_steps, sample_what=sample_what)


# config 5 block: 8 x 2048 tokens, d_model 1024, 16 heads x 64, FFN 4096
_C5_TOK = 8 * 2048
_C5_MM_FLOPS = 2 * _C5_TOK * (4 * 1024 * 1024 + 2 * 1024 * 4096)
_C5_ATT_FLOPS = 2 * 2 * 8 * 16 * 2048 * 2048 * 64 // 2          # QK^T and PV, causal half
# config 3 step: forward + dX (layers 2,3) + dW (all), batch 8192, 1024-4096-4096-1024
_C3_FLOPS = 2 * 8192 * (1024 * 4096 + 4096 * 4096 + 4096 * 1024) * 3 - 2 * 8192 * 1024 * 4096

WORKLOADS = {
    "c2_f32": _wl("c2_chain_f32", "eltwise HBM GB/s", "GB/s", 7 * N_C2 * 4 + 2 * 4096 * 4, 1e9, "hbm", "f32",
                  "config 2: LayerNorm -> tanh-GELU -> softmax -> full sum on f32 (8192,4096); "
                  "bytes = LayerNorm r+w, GELU r+w, softmax r+w, sum r, + gamma/beta",
                  sample="c2_chain_f32_cpu_sample", sample_frac=512 / 8192, traffic=778.3e6,
                  sample_what="512 of the 8192 rows"),
    "c2_bf16": _wl("c2_chain_bf16", "eltwise HBM GB/s", "GB/s", 7 * N_C2 * 2 + 2 * 4096 * 2, 1e9, "hbm", "bf16",
                   "config 2 on bf16-storage copies of the same values",
                   sample="c2_chain_bf16_cpu_sample", sample_frac=512 / 8192, sample_what="512 of the 8192 rows"),
    "c2_i32": _wl("c2_int_chain", "eltwise HBM GB/s", "GB/s", 5 * N_C2 * 4, 1e9, "hbm", "i32",
                  "config 2: max((a+b)^c, d) on i32 (8192,4096), bit-exact",
                  sample="c2_int_chain_cpu_sample", sample_frac=512 / 8192, sample_what="512 of the 8192 rows"),
    "dot_bf16_8192": _wl("dot_bf16_8192", "dot_general TFLOP/s", "TFLOP/s", 2 * 8192 ** 3, 1e12, "tensor", "bf16",
                         "one dot_general bf16 8192 x 8192 x 8192, f32 accumulate, bf16 result"),
    "dot_bf16_4096": _wl("dot_bf16_4096", "dot_general TFLOP/s", "TFLOP/s", 2 * 4096 ** 3, 1e12, "tensor", "bf16",
                         "one dot_general bf16 4096 x 4096 x 4096", secondary=True, traffic=163.1e6),
    "flash_bf16": _wl("flash_bf16_c5", "flash-attention TFLOP/s", "TFLOP/s", _C5_ATT_FLOPS, 1e12, "tensor", "bf16",
                      "config 5's attention alone: 128 heads x 2048 x 2048, head_dim 64, causal (flops count the "
                      "causal half)", secondary=True, traffic=150.6e6),
    "c3_mlp": _wl("c3_mlp_step_bf16", "dot_general TFLOP/s", "TFLOP/s", _C3_FLOPS, 1e12, "tensor", "bf16",
                  "config 3: 3-layer MLP forward + grad of MSE + SGD step, batch 8192, 1024-4096-4096-1024, bf16; "
                  "on N GPUs: local-batch gradients, NCCL all-reduce, SGD program", plan="c3"),
    "c5_block": _wl("c5_block_bf16", "transformer-block tokens/s per B200", "tokens/s", _C5_TOK, 1.0, "tensor", "bf16",
                    "config 5: pre-norm decoder block forward, batch 8 x seq 2048, d_model 1024, 16 x 64 heads, "
                    "causal flash attention, GELU FFN 4096, bf16",
                    roof_alg=_C5_MM_FLOPS + _C5_ATT_FLOPS, plan="c5_block", traffic=1139.5e6,
                    sample="c5_block_bf16_cpu_sample", sample_frac=512 / _C5_TOK,
                    sample_what="one sequence of 512 tokens through the same block (8 x 2048 in the workload)"),
    "c4_nbody": _wl("c4_nbody", "n-body pair interactions/s", "G interactions/s", 4096 * 4096 * 4 * 200, 1e9, "hbm",
                    "f32", "config 4: 4096 bodies, RK4, 200 steps in one FOR loop (one system per GPU), executed as "
                    "the decomposed bytecode, whose (N,N,3) intermediates make it HBM-bound; bytes per step = the "
                    "tile ops' inputs + outputs over the four acceleration evaluations, A = 201 MB (N,N,3) and "
                    "B = 67 MB (N,N) tensors: 28 A + 16 B",
                    roof_alg=(28 * 4096 * 4096 * 3 * 4 + 16 * 4096 * 4096 * 4) * 200, secondary=True, plan="c4",
                    max_steps=3),
    "c4_nbody_2steps": _wl("c4_nbody_2steps", "n-body pair interactions/s", "G interactions/s", 4096 * 4096 * 4 * 2, 1e9, "hbm",
                           "f32", "config 4 cut to 2 RK4 steps (46 grid barriers): the same phases as the 200-step launch, "
                           "short enough to profile", roof_alg=(28 * 4096 * 4096 * 3 * 4 + 16 * 4096 * 4096 * 4) * 2,
                           secondary=True),
    "c3_stage_gelu_grad": _wl("c3_stage_gelu_grad_f32", "eltwise HBM GB/s", "GB/s", 2 * N_C2 * 4, 1e9, "hbm", "f32",
                              "config 3 stage: the GELU-derivative MAP_REGION (14 micro-ops) over 8192 x 4096 f32",
                              secondary=True),
    "flash_decode_bf16": _wl("flash_decode_bf16_c5", "decode-attention GB/s", "GB/s", 2 * 512 * 2049 * 64 * 2, 1e9, "hbm", "bf16",
                             "config 5's decode attention alone: 512 heads x 1 query x 2049 keys, head_dim 64; "
                             "bytes = K and V read once", secondary=True, traffic=283.2e6),
    "c5_decode_in_place": _wl("c5_decode_in_place_bf16", "transformer-block tokens/s per B200", "tokens/s", 32, 1.0, "hbm", "bf16",
                              "config 5 decode step, batch 32, KV cache 2048 + the new position: K/V written in place "
                              "(in/out buffers), K read through its view; bytes = weights + KV cache read once",
                              roof_alg=2 * (4 * 1024 * 1024 + 2 * 1024 * 4096) + 2 * 32 * 16 * 2049 * 64 * 2,
                              plan="c5_decode_in_place", traffic=310.5e6),
    "c5_decode": _wl("c5_decode_bf16", "transformer-block tokens/s per B200", "tokens/s", 32, 1.0, "hbm", "bf16",
                     "config 5 decode step: batch 32, KV cache 2048; bytes = weights + KV cache read once",
                     roof_alg=2 * (4 * 1024 * 1024 + 2 * 1024 * 4096) + 2 * 32 * 16 * 2048 * 64 * 2, plan="c5_decode"),
}


# the stages of config 2 on their own: one tile-op family per program
for _stage, _bytes, _what in (
        ("layernorm", 2 * N_C2 * 4, "LAYERNORM_SEG rows of 4096 (TMA-staged)"),
        ("affine_gelu", 2 * N_C2 * 4 + 2 * 4096 * 4, "fused chain mul(gamma view), add(beta view), GELU"),
        ("softmax", 2 * N_C2 * 4, "SOFTMAX_SEG rows of 4096 (TMA-staged)"),
        ("sum", N_C2 * 4, "full sum: RED_PART + RED_COMB")):
    WORKLOADS[f"c2_stage_{_stage}"] = _wl(f"c2_stage_{_stage}_f32", "eltwise HBM GB/s", "GB/s", _bytes, 1e9, "hbm",
                                          "f32", f"config 2 stage: {_what}", secondary=True)


def load_blob(name: str) -> bytes:
    with gzip.open(os.path.join(PROG_DIR, name + ".vmprog.gz"), "rb") as f:
        return f.read()


def manifest():
    return json.load(open(os.path.join(PROG_DIR, "manifest.json")))


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nme, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nme)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_arm(w: dict, steps: int, warmup: int, threads: int, budget_s: float = 200.0):
    """Time the CPU arm on the workload's bounded sample: every step executes the whole
    sample program once. Returns (metric value, seconds per step, steps actually timed).
    The steps are cut short (and the count returned says so) only if they would not fit
    `budget_s` seconds."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import vmoracle
    man = manifest()[w["sample"]]
    blob = load_blob(w["sample"])
    args = gen_inputs.gen_all(man["seed"], man["items"])
    prog = vmoracle.Program(blob)
    t0 = time.perf_counter()
    prog.execute(args, threads=threads)                      # first call also builds / loads the library
    first = time.perf_counter() - t0
    for _ in range(max(0, min(warmup, int(budget_s * 0.2 / max(first, 1e-6))) - 1)):
        prog.execute(args, threads=threads)
    steps = max(1, min(steps, int(budget_s * 0.8 / max(first, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(steps):
        prog.execute(args, threads=threads)
    dt = (time.perf_counter() - t0) / steps
    return w["alg"] * w["sample_frac"] / dt / w["scale"], dt, steps


def oracle_rows(sample_program, x_rows, gamma, beta):
    """Config 2 on a row sample through the C oracle (the checker of `verified`)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import vmoracle
    return vmoracle.Program(load_blob(sample_program)).execute([np.ascontiguousarray(x_rows), gamma, beta])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c5_block", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-verify", action="store_true", help="skip the value check of the last step's results")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = WORKLOADS[a.workload]
    if w["max_steps"]:
        a.steps, a.warmup = min(a.steps, w["max_steps"]), min(a.warmup, 3)
    cores = os.cpu_count() or 1
    base = {"metric": w["metric"], "unit": w["unit"], "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": a.workload, "what": w["desc"], "program": w["program"],
                       "lanes": 148, "ew_tile": 4096, "l2": ""}}

    if a.impl == "reference":
        if rank != 0:
            return
        if not w["sample"]:
            print(json.dumps({"impl": "reference", "unavailable": f"no bounded CPU sample is defined for workload {a.workload}"}))
            return
        val, dt, steps = cpu_arm(w, a.steps, a.warmup, cores)
        sample = f"{w['sample']}: {w['sample_what']}; every step runs the whole sample once ({dt:.2f} s)"
        cfg = dict(base["config"], sample=sample)
        line = dict(base, config=cfg, impl="reference", value=val, steps=steps, ms_per_step=dt * 1e3,
                    cpu_baseline={"value": val, "unit": w["unit"], "cores": cores, "kind": "port", "sample": sample},
                    e2e={"value": val, "unit": w["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0,
                    note="reference device kernels are OpenCL C (no OpenCL runtime, no jax on this box): the CPU arm is the "
                         "C restatement of its per-phase host walk and CPU tile bodies, OpenMP over all host cores; "
                         "the full workload does not fit a sensible time on it, so a step is the bounded sample named in config"
                         + ("" if steps == a.steps else f"; {steps} of the {a.steps} requested steps fit the time budget"))
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    vm = importlib.import_module("pjrt-ocl_b200")
    rt = vm.Runtime.Create(local_rank)
    # a non-default stream: its handle is what the C ABI launches on, and what the
    # timing events are recorded on
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)

    dp = importlib.import_module("pjrt-ocl_b200.dataparallel")

    l2_note = [""]

    def run_workload(wl: dict, steps: int, warmup: int, want_e2e: bool):
        plan = dp.PLANS.get(wl["plan"]) if wl["plan"] else None
        name = plan.rank_program(world) if plan else wl["program"]
        man = manifest()[name]
        lp = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(load_blob(name)))
        host_in = [np.ascontiguousarray(x) for x in gen_inputs.gen_all(man["seed"] + (rank if plan and plan.seed_per_rank else 0), man["items"])]
        if plan and world > 1:
            # inputs listed at the global batch are sliced; per-shard listings already have the local shape
            host_in = [dp.shard_rows(x, rank, world) if (i in plan.batch_inputs and x.nbytes != lp.prog.inputs[i]["bytes"])
                       else x for i, x in enumerate(host_in)]
        pin_in = []
        for x in host_in:
            t = torch.empty(max(x.nbytes, 1), dtype=torch.uint8, pin_memory=True)
            t[:x.nbytes] = torch.from_numpy(x.reshape(-1).view(np.uint8))
            pin_in.append(t)
        dev_in = [t.cuda(non_blocking=True) for t in pin_in]
        # results of a data-parallel step that are summed over ranks live back to back in ONE buffer,
        # so the exchange is a single all-reduce (16-byte aligned slots; the program writes into them)
        bucket, bucket_slots = None, {}
        if world > 1 and plan and len(plan.reduce_outputs) > 1:
            off = 0
            for i in plan.reduce_outputs:
                bucket_slots[i] = off
                off += (lp.prog.outputs[i]["bytes"] + 15) // 16 * 16
            bucket = torch.zeros(off, dtype=torch.uint8, device="cuda")
        dev_out = [bucket[bucket_slots[i]:bucket_slots[i] + max(s["bytes"], 16)] if i in bucket_slots
                   else torch.empty(max(s["bytes"], 16), dtype=torch.uint8, device="cuda")
                   for i, s in enumerate(lp.prog.outputs)]
        # in/out buffers (a KV cache updated in place): the result is the argument's own memory
        for i_arg, i_res in lp.InOutResults().items():
            dev_out[i_res] = dev_in[i_arg]
        pin_out = [torch.empty(max(s["bytes"], 1), dtype=torch.uint8, pin_memory=True) for s in lp.prog.outputs]
        torch.cuda.synchronize()
        ins = [t.data_ptr() for t in dev_in]
        outs = [t.data_ptr() for t in dev_out]
        # the exchange step of the configuration, if it has one (NCCL, on the launching stream)
        reduce_views, lp2, ins2, outs2, dev_out2 = [], None, None, None, None
        if world > 1:
            if bucket is not None:
                reduce_views = [bucket.view(torch.float32)]          # padding between slots is zero on every rank
            elif plan and plan.reduce_outputs:
                reduce_views = [dev_out[i][:lp.prog.outputs[i]["bytes"]].view(torch.float32) for i in plan.reduce_outputs]
            elif wl["program"].startswith("c2_chain"):
                reduce_views = [dev_out[-1][:4].view(torch.float32)]
            if plan and plan.apply_program:
                lp2 = vm.LoadedProgram.Load(rt, vm.VmProgram.Parse(load_blob(plan.apply_program)))
                dev_out2 = [torch.empty(max(s["bytes"], 16), dtype=torch.uint8, device="cuda") for s in lp2.prog.outputs]
                ins2 = [ins[i] for i in plan.apply_inputs] + [outs[i] for i in plan.reduce_outputs[plan.apply_skip:]]
                outs2 = [t.data_ptr() for t in dev_out2]

        def step():
            lp.ExecuteDeviceAsync(ins, outs, stream.cuda_stream)
            for v in reduce_views:
                dist.all_reduce(v)
            if lp2 is not None:
                lp2.ExecuteDeviceAsync(ins2, outs2, stream.cuda_stream)

        def every_rank(cond: bool) -> bool:
            # the same answer on all ranks: the loops below hold steps with collectives in them
            return dp.ranks_agree(cond, "cuda")

        sampler = ClockSampler(local_rank)
        sampler.start()
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        if want_e2e:
            # nvidia-smi needs most of a second before its first sample: keep the same load running until it
            # reports, so that the clock record covers the timed region that follows
            t_soak = time.perf_counter()
            while every_rank(not sampler.lines and time.perf_counter() - t_soak < 2.0):
                for _ in range(8):
                    step()
                torch.cuda.synchronize()
        st = lp.Status()
        phases = lp.PhaseTimes()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        launches0 = lp.launch_count + (lp2.launch_count if lp2 else 0)
        # L2 hygiene: a workload whose arguments fit the 126 MB L2 gets the cache flushed between timed
        # steps (a 256 MB fill), each step then timed by its own pair of events; larger ones run back to back
        in_bytes = sum(x.nbytes for x in host_in)
        flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if in_bytes < (252 << 20) else None
        l2_note[0] = ("flushed between timed steps (256 MB fill; arguments total %.0f MB)" % (in_bytes / 1e6)
                      if flush_buf is not None else "arguments larger than L2 (%.0f MB), steps back to back" % (in_bytes / 1e6))
        if flush_buf is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                step()
            e1.record(stream)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        else:
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            for b0, b1 in evs:
                flush_buf.fill_(1)
                b0.record(stream)
                step()
                b1.record(stream)
            torch.cuda.synchronize()
            ms = sum(b0.elapsed_time(b1) for b0, b1 in evs)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        del flush_buf
        lp.Status()
        launches = lp.launch_count + (lp2.launch_count if lp2 else 0) - launches0
        if want_e2e:
            # the timed region of a short run fits between two samples: the same steps continue (untimed)
            # until the sampler has seen at least 0.3 s of this load
            t_soak = time.perf_counter()
            while every_rank(time.perf_counter() - t_soak < max(0.0, 0.3 - ms * 1e-3)):
                for _ in range(8):
                    step()
                torch.cuda.synchronize()
        clocks = sampler.stop()
        clocks["window"] = "timed region + identical untimed continuation to >= 0.3 s under load"
        # where one step's time goes: CUDA events around the program(s) and the exchange
        stages = None
        if want_e2e and world > 1 and (reduce_views or lp2 is not None):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record(stream)
            lp.ExecuteDeviceAsync(ins, outs, stream.cuda_stream)
            ev[1].record(stream)
            for v in reduce_views:
                dist.all_reduce(v)
            ev[2].record(stream)
            if lp2 is not None:
                lp2.ExecuteDeviceAsync(ins2, outs2, stream.cuda_stream)
            ev[3].record(stream)
            torch.cuda.synchronize()
            stages = {"program_ms": ev[0].elapsed_time(ev[1]), "all_reduce_ms": ev[1].elapsed_time(ev[2]),
                      "apply_program_ms": ev[2].elapsed_time(ev[3]),
                      "all_reduce_bytes": int(sum(v.numel() * 4 for v in reduce_views))}
        # value check of the last step's results (this rank's shard)
        verified, verified_what = None, ""
        if want_e2e and not a.no_verify:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import fullsize_refs
            torch.cuda.synchronize()
            try:
                if lp2 is None:
                    host_out = [d.cpu().numpy()[:s["bytes"]] for d, s in zip(dev_out, lp.prog.outputs)]
                    replica_sums = []       # replicas of one input: an all-reduced result is `world` times the single-GPU value
                    if world > 1 and plan and plan.reduce_outputs and not plan.batch_inputs and not plan.seed_per_rank:
                        replica_sums = list(plan.reduce_outputs)
                    elif world > 1 and not plan and wl["program"].startswith("c2_chain"):
                        replica_sums = [len(host_out) - 1]
                    for i in replica_sums:
                        host_out[i] = (host_out[i].view(np.float32) / np.float32(world)).view(np.uint8)
                    verified_what = fullsize_refs.verify_workload(name, host_in, host_out, oracle_rows)
                    if replica_sums and verified_what:
                        verified_what += f"; the all-reduced scalar is {world} x the single-GPU one"
                else:
                    # config 3 on N GPUs: every rank must hold the same updated weights, and they must be
                    # what the single-GPU step gives on the global batch (checked on rank 0)
                    host_out = [d.cpu().numpy()[:s["bytes"]] for d, s in zip(dev_out2, lp2.prog.outputs)]
                    crc = torch.tensor([float(int(np.bitwise_xor.reduce(np.concatenate([h.view(np.uint8) for h in host_out]).view(np.uint32))))],
                                       dtype=torch.float64, device="cuda")
                    lo_, hi_ = crc.clone(), crc.clone()
                    dist.all_reduce(lo_, op=dist.ReduceOp.MIN)
                    dist.all_reduce(hi_, op=dist.ReduceOp.MAX)
                    assert float(lo_.item()) == float(hi_.item()), "ranks disagree on the updated weights"
                    if rank == 0:
                        full_in = [np.ascontiguousarray(x) for x in gen_inputs.gen_all(man["seed"], man["items"])]
                        loss = dev_out[0][:4].cpu().numpy()
                        verified_what = fullsize_refs.verify_workload("c3_mlp_step", full_in, [loss] + host_out)
                    verified_what = (verified_what or "as rank 0") + "; all ranks hold identical weights"
                verified = True if verified_what else None     # None: no value check exists for this workload
            except AssertionError as e:
                verified, verified_what = False, (str(e)[:300] or "a value check failed (bare assertion in tests/fullsize_refs.py)")
        e2e = None
        if want_e2e:
            n_e2e = max(3, min(steps, 10))
            h2d = int(sum(x.nbytes for x in host_in))
            d2h = int(sum(s["bytes"] for s in lp.prog.outputs))
            if world == 1:
                # the call a user makes: host arrays in, host arrays out (copies inside)
                np_in = [t.numpy()[:x.nbytes].view(x.dtype).reshape(x.shape) for t, x in zip(pin_in, host_in)]
                np_out = [t.numpy()[:s["bytes"]] for t, s in zip(pin_out, lp.prog.outputs)]
                for _ in range(2):
                    lp.Execute(np_in, out=np_out)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(n_e2e):
                    lp.Execute(np_in, out=np_out)
                dt = (time.perf_counter() - t0) / n_e2e
            else:
                # per rank: pinned inputs -> device, the data-parallel step, first result -> pinned host
                src = dev_out2 if dev_out2 is not None else dev_out
                pin_res = [torch.empty(d.numel(), dtype=torch.uint8, pin_memory=True) for d in src]

                def e2e_step():
                    for d, p_ in zip(dev_in, pin_in):
                        d.copy_(p_, non_blocking=True)
                    step()
                    for p_, d in zip(pin_res, src):
                        p_.copy_(d, non_blocking=True)
                    torch.cuda.synchronize()
                for _ in range(2):
                    e2e_step()
                dist.barrier()
                t0 = time.perf_counter()
                for _ in range(n_e2e):
                    e2e_step()
                dt = (time.perf_counter() - t0) / n_e2e
                if dev_out2 is not None:
                    d2h = int(sum(s["bytes"] for s in lp2.prog.outputs))
            e2e = {"seconds": dt, "h2d": h2d, "d2h": d2h, "steps": n_e2e}
        if lp2 is not None:
            lp2.close()
        st["tensor_core_matmuls"] = [lp.stat("tensor_core_matmuls"), lp.stat("matmuls")]
        lp.close()
        st["phase_ns"] = phases
        st["stages"] = stages
        st["verified"] = verified
        st["verified_what"] = verified_what
        return ms / steps, launches, clocks, e2e, st

    ms_step, launches, clocks, e2e, st = run_workload(w, a.steps, a.warmup, True)
    base["config"]["l2"] = l2_note[0]
    t_max = torch.tensor([ms_step], device="cuda")
    e2e_t = torch.tensor([e2e["seconds"]], device="cuda")
    if world > 1:
        dist.all_reduce(t_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    ms_step = float(t_max.item())
    plan = dp.PLANS.get(w["plan"]) if w["plan"] else None
    strong = bool(plan and plan.scaling == "strong")
    total_alg = w["alg"] if strong else w["alg"] * world          # strong scaling: the global batch is fixed
    value = total_alg / (ms_step * 1e-3) / w["scale"]
    base["scaling"] = "strong" if strong else "weak"
    base["config"]["parallelism"] = ("single GPU" if world == 1 else
                                     f"dp{world}: {'batch shards' if strong else 'one independently seeded system per GPU' if plan and plan.seed_per_rank else 'replicas'}"
                                     + (", NCCL all-reduce between the gradient and SGD programs" if plan and plan.apply_program else
                                        ", scalar all-reduce" if w["program"].startswith("c2_chain") else ", no exchange step"))
    roof_scale = 1e9 if w["bound"] == "hbm" else 1e12
    achieved = (w["roof_alg"] / world if strong else w["roof_alg"]) / (ms_step * 1e-3) / roof_scale   # per GPU

    extra = {}
    if not a.no_extra:
        # N = 1: every other workload; N > 1: the two batch-sharded configurations (all ranks take part)
        names = [n for n in WORKLOADS if n != a.workload] if world == 1 else \
                [n for n in ("c5_block", "c3_mlp") if n != a.workload]
        for name in names:
            wl = WORKLOADS[name]
            m, _, _, _, _ = run_workload(wl, min(max(5, min(a.steps // 2, 100)), wl["max_steps"] or 100),
                                         1 if wl["max_steps"] else 3, False)
            tm = torch.tensor([m], device="cuda")
            if world > 1:
                dist.all_reduce(tm, op=dist.ReduceOp.MAX)
            m = float(tm.item())
            pl = dp.PLANS.get(wl["plan"]) if wl["plan"] else None
            tot = wl["alg"] if (pl and pl.scaling == "strong") else wl["alg"] * world
            strong_x = bool(pl and pl.scaling == "strong")
            ach = (wl["roof_alg"] / world if strong_x else wl["roof_alg"]) / (m * 1e-3) / (1e9 if wl["bound"] == "hbm" else 1e12)
            extra[name] = {wl["unit"]: tot / (m * 1e-3) / wl["scale"], "ms_per_step": m,
                           "scaling": "strong" if strong_x else "weak",
                           "roofline": {"bound": wl["bound"], "achieved": ach, "unit": "GB/s" if wl["bound"] == "hbm" else "TFLOP/s"}}

    ver = torch.tensor([1.0 if st["verified"] else 0.0 if st["verified"] is not None else 2.0], device="cuda")
    if world > 1:
        dist.all_reduce(ver, op=dist.ReduceOp.MIN)
    verified = None if float(ver.item()) == 2.0 else float(ver.item()) == 1.0
    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        key = "hbm_gbs" if w["bound"] == "hbm" else "bf16_tflops"
        if os.path.exists(peaks_path):
            pk = json.load(open(peaks_path))
            peak, peak_src = pk[key], f"measured (MEASURED_PEAKS.json {key})"
            for e in extra.values():
                e["roofline"]["frac"] = e["roofline"]["achieved"] / pk["hbm_gbs" if e["roofline"]["bound"] == "hbm" else "bf16_tflops"]
        else:
            peak, peak_src = (6650.0 if w["bound"] == "hbm" else 1590.0), "fallback"
            for e in extra.values():
                e["roofline"]["frac"] = e["roofline"]["achieved"] / (6650.0 if e["roofline"]["bound"] == "hbm" else 1590.0)
        cpu = None
        if world == 1 and w["sample"]:
            cv, cdt, csteps = cpu_arm(w, 3, 1, cores, budget_s=40.0)
            cpu = {"value": cv, "unit": w["unit"], "cores": cores, "kind": "port",
                   "sample": f"{w['sample']}: {w['sample_what']}, {csteps} steps, {cdt:.2f} s each"}
        line = dict(base, value=value, ms_per_step=ms_step, clocks=clocks, gpu_launches=launches,
                    e2e={"value": total_alg / float(e2e_t.item()) / w["scale"], "unit": w["unit"],
                         "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
                    roofline={"bound": w["bound"], "achieved": achieved, "peak": peak,
                              "unit": "GB/s" if w["bound"] == "hbm" else "TFLOP/s",
                              "frac": achieved / peak, "traffic": w["traffic"], "peak_source": peak_src,
                              "kernel": "b2_vm<512> (one launch per step)"},
                    cpu_baseline=cpu, device_ns_per_step=st["device_ns"], grid_barriers=st["barriers"],
                    phase_end_ns=st["phase_ns"], tensor_core_matmuls=st["tensor_core_matmuls"],
                    verified=verified, verified_what=st["verified_what"], stages_ms=st["stages"],
                    other_workloads=extra)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
