#!/usr/bin/env python
"""Assemble the benchmark programs (the five configurations at their full sizes,
148 lanes, EW tile 4096, matmul tile 128) into pjrt-ocl_b200/programs/*.vmprog.gz
plus a JSON manifest describing their seeded inputs.

Build-time only: needs the reference checkout on PYTHONPATH
(PYTHONPATH=<reference>/python python pjrt-ocl_b200/programs/make_programs.py).
The blobs are what the reference's lowering + scheduler emit for these graphs;
the device executes them unchanged.
"""
from __future__ import annotations

import gzip
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import cases  # noqa: E402
from vmasm import BF16, F32  # noqa: E402

# Programs whose phases hold several equal units (the three q/k/v projections, the three
# head transposes): the scheduler gives each unit ceil(lanes * share) chunks, which for
# 148 lanes and three units is 150 chunks - two lanes would run two chunks and the phase
# twice as long. 144 divides by 2, 3, 4, 6 and 8.
MULTI_UNIT_LANES = 144

PROGRAMS = {
    "c1_relu_matmul": lambda: cases.c1_relu_matmul(),
    "c2_chain_f32": lambda: cases.c2_chain(dtype=F32),
    "c2_chain_bf16": lambda: cases.c2_chain(dtype=BF16),
    "c2_chain_f32_decomposed": lambda: cases.c2_chain(dtype=F32, fused=False),
    "c2_int_chain": lambda: cases.c2_int_chain(),
    "c3_mlp_step_bf16": lambda: cases.c3_mlp_step(nlanes=MULTI_UNIT_LANES),
    "c4_nbody": lambda: cases.c4_nbody(),
    "c5_block_bf16": lambda: cases.c5_block(nlanes=MULTI_UNIT_LANES),
    "c5_decode_bf16": lambda: cases.c5_decode(nlanes=MULTI_UNIT_LANES),
    "c5_decode_in_place_bf16": lambda: cases.c5_decode_in_place(nlanes=MULTI_UNIT_LANES),
}
# data-parallel shards of config 3 / 5 (batch split over 2, 4, 8 GPUs)
for g in (2, 4, 8):
    PROGRAMS[f"c3_mlp_grads_bf16_dp{g}"] = (
        lambda g=g: cases.c3_mlp_step(batch=8192 // g, global_batch=8192, apply_sgd=False, nlanes=MULTI_UNIT_LANES))
    PROGRAMS[f"c5_block_bf16_dp{g}"] = lambda g=g: cases.c5_block(batch=8 // g, nlanes=MULTI_UNIT_LANES)
    PROGRAMS[f"c5_decode_bf16_dp{g}"] = lambda g=g: cases.c5_decode(batch=32 // g, nlanes=MULTI_UNIT_LANES)
    PROGRAMS[f"c5_decode_in_place_bf16_dp{g}"] = (
        lambda g=g: cases.c5_decode_in_place(batch=32 // g, nlanes=MULTI_UNIT_LANES))
# the four stages of config 2 as programs of their own (one tile-op family each),
# for per-family roofline numbers and ncu captures
for stage in ("layernorm", "affine_gelu", "softmax", "sum"):
    PROGRAMS[f"c2_stage_{stage}_f32"] = lambda stage=stage: cases.c2_stage(stage)
# bounded samples of config 2 (512 of the 8192 rows) for the timed CPU arm
PROGRAMS["c2_chain_f32_cpu_sample"] = lambda: cases.c2_chain(rows=512, dtype=F32)
PROGRAMS["c2_chain_bf16_cpu_sample"] = lambda: cases.c2_chain(rows=512, dtype=BF16)
PROGRAMS["c2_int_chain_cpu_sample"] = lambda: cases.c2_int_chain(rows=512)
# bounded sample of config 5 for the timed CPU arm: one sequence of 512 tokens through the same block
PROGRAMS["c5_block_bf16_cpu_sample"] = lambda: cases.c5_block(batch=1, seq=512, nlanes=16)
PROGRAMS["c3_sgd_apply_bf16"] = lambda: cases.sgd_apply(
    [(1024, 4096), (4096, 4096), (4096, 1024)])


# the matmul tile-op family on its own
# config 4 at its full 4096 bodies but two RK4 steps: small enough in time for a float64
# recomputation on the host (the full-size parity case; the 200-step program is the bench)
PROGRAMS["c4_nbody_2steps"] = lambda: cases.c4_nbody(steps=2)
PROGRAMS["dot_bf16_8192"] = lambda: cases.dot_general_square(8192)
PROGRAMS["dot_bf16_4096"] = lambda: cases.dot_general_square(4096)
PROGRAMS["flash_bf16_c5"] = lambda: cases.flash_only()
PROGRAMS["flash_decode_bf16_c5"] = lambda: cases.flash_decode_only()
PROGRAMS["c3_stage_gelu_grad_f32"] = lambda: cases.region_only()


def main():
    sel = sys.argv[1:]
    manifest_path = os.path.join(HERE, "manifest.json")
    manifest = json.load(open(manifest_path)) if os.path.exists(manifest_path) else {}
    for name, fn in PROGRAMS.items():
        if sel and not any(s in name for s in sel):
            continue
        blob, prog, spec = fn()
        with gzip.GzipFile(os.path.join(HERE, name + ".vmprog.gz"), "wb", mtime=0) as f:
            f.write(blob)
        manifest[name] = {
            "seed": spec[0] if spec else None, "items": spec[1] if spec else None,
            "arena_bytes": prog.arena_bytes, "n_instrs": len(prog.instrs),
            "blob_bytes": len(blob),
        }
        print(f"{name:34s} blob {len(blob):9d} B  arena {prog.arena_bytes / 2**20:10.1f} MiB")
    json.dump(manifest, open(manifest_path, "w"), indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
