"""Data-parallel execution of batch-sharded programs: one process and one
megakernel per GPU, the exchange step (if the configuration has one) on NCCL.

The reference has no multi-device path; its programs are single-device. What is
sharded here is the *configuration*: the same graph compiled for the local batch
(`<program>_dp<N>`), inputs sliced along the batch axis, and - only where the
graph has a cross-batch reduction (config 3's weight gradients, config 2's final
scalar) - an all-reduce between the program that produces the partial result and
the program that consumes it.

Everything here is host logic over two callables, so it runs unchanged on the
CUDA runtime (NCCL) and, in the CPU tests, on the oracle with gloo.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional, Sequence

import numpy as np


def ranks_agree(cond: bool, device=None) -> bool:
    """`cond` or-ed over all ranks of the default process group (just `cond` without one). A loop whose body holds
    collectives must run the same number of times on every rank, so it may not end on a rank's own clock or
    sampler: every rank asks this instead, once per iteration."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return bool(cond)
    flag = torch.tensor([1 if cond else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return bool(flag.item())


def shard_rows(arr: np.ndarray, rank: int, world: int) -> np.ndarray:
    """Rank `rank`'s rows of a batch-major array (the batch must divide evenly)."""
    n = arr.shape[0]
    if n % world:
        raise ValueError(f"batch {n} does not divide over {world} ranks")
    per = n // world
    return np.ascontiguousarray(arr[rank * per:(rank + 1) * per])


@dataclasses.dataclass(frozen=True)
class DpPlan:
    """How one configuration runs on `world` GPUs.

    program:       name of the single-GPU program (world == 1)
    dp_program:    name pattern of the per-rank program, `{n}` = world (None: replicate `program`)
    batch_inputs:  indices of inputs that are sliced along axis 0 (the rest are replicated)
    reduce_outputs: indices of the per-rank program's outputs that are summed over ranks
    apply_program: program run after the reduction (None: none); its inputs are
                   `apply_inputs` (indices into the per-rank INPUTS) followed by the
                   reduced outputs in `reduce_outputs[apply_skip:]` order
    seed_per_rank: every rank draws its own inputs (seed + rank): independent units, nothing shared
    """
    program: str
    dp_program: Optional[str] = None
    batch_inputs: Sequence[int] = ()
    reduce_outputs: Sequence[int] = ()
    apply_program: Optional[str] = None
    apply_inputs: Sequence[int] = ()
    apply_skip: int = 0
    scaling: str = "weak"
    seed_per_rank: bool = False

    def rank_program(self, world: int) -> str:
        if world == 1 or self.dp_program is None:
            return self.program
        return self.dp_program.format(n=world)


PLANS = {
    # config 2: replicas; the final scalar is summed over ranks
    "c2": DpPlan("c2_chain_f32", reduce_outputs=(1,), scaling="weak"),
    # config 3: gradients of the local batch, summed, then one SGD step on every rank
    "c3": DpPlan("c3_mlp_step_bf16", "c3_mlp_grads_bf16_dp{n}", batch_inputs=(0, 1), reduce_outputs=(0, 1, 2, 3),
                 apply_program="c3_sgd_apply_bf16", apply_inputs=(2, 3, 4), apply_skip=1, scaling="strong"),
    # config 4: one independent system (seed) per GPU, no exchange
    "c4": DpPlan("c4_nbody", seed_per_rank=True, scaling="weak"),
    # config 5: batch shards, no exchange
    "c5_block": DpPlan("c5_block_bf16", "c5_block_bf16_dp{n}", scaling="strong"),
    "c5_decode": DpPlan("c5_decode_bf16", "c5_decode_bf16_dp{n}", scaling="strong"),
    "c5_decode_in_place": DpPlan("c5_decode_in_place_bf16", "c5_decode_in_place_bf16_dp{n}", scaling="strong"),
}


def rank_inputs(plan: DpPlan, inputs: Sequence[np.ndarray], rank: int, world: int) -> list:
    """The per-rank program's inputs, from inputs drawn at the global batch."""
    if world == 1:
        return list(inputs)
    return [shard_rows(a, rank, world) if i in plan.batch_inputs else a for i, a in enumerate(inputs)]


def step(plan: DpPlan, world: int, run: Callable[[str, list], list], all_reduce_sum: Callable[[np.ndarray], np.ndarray],
         inputs: list) -> list:
    """One data-parallel step on this rank. `run(program_name, inputs) -> outputs`
    executes a program; `all_reduce_sum(array) -> array` sums over ranks. Returns the
    step's results: the apply program's outputs preceded by the reduced outputs it
    does not consume (config 3: loss, then the three updated weights - the same
    list the single-GPU program returns)."""
    outs = run(plan.rank_program(world), inputs)
    if world > 1:
        outs = list(outs)
        for i in plan.reduce_outputs:
            outs[i] = all_reduce_sum(outs[i])
        if plan.apply_program:
            red = [outs[i] for i in plan.reduce_outputs]
            applied = run(plan.apply_program, [inputs[i] for i in plan.apply_inputs] + red[plan.apply_skip:])
            return red[:plan.apply_skip] + list(applied)
    return list(outs)
