"""Thresholds that were found by measurement, in one place.

Each of them chooses between kernels that compute the same thing, so a wrong value costs time, never
correctness.  They were measured on one B200 with the layer sizes of Qwen1.5-MoE-A2.7B (hidden 2048,
60 experts of 1408 with top-4 routing, shared expert 5632, 16 heads of 128) and checked at
Qwen2-57B-A14B sizes; another width, expert count or GPU should re-measure them (``bench.py
--point-batches`` walks the batch sizes around each threshold) rather than inherit them silently.
``TUNING`` is the instance the parts read; a host program may replace its fields before it loads a model.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass
class Tuning:
    # Dense products (o_proj, shared expert, dense MLP, output head) of steps with at most this many tokens
    # run on the engine's own decode kernel, which streams the weights once with 16 features per block;
    # above it the library product is used.  The four thresholds of the "smallest steps" (this one, the shared
    # expert forked after the routing, the L2 hints and dependent launch) moved together from 8 to 15 tokens:
    # batch 9 +6 % (a step of 9 had been slower per token than a step of 8), 12 +6 %, 15 +4 %; at 16 tokens
    # and above, where the expert products change to the tcgen05 kernel, the same settings lose 4 to 9 %.
    dense_skinny_max_tokens: int = 15

    # Grouped expert products of steps above 8 tokens: up to this many rows per expert on average (tokens *
    # top_k / experts) the decode-sized mma.sync kernel reads every used expert once into fragments; above it
    # the persistent tcgen05 kernel, whose TMA ring keeps four times as many bytes in flight, streams the same
    # weights faster even though its tiles are nearly empty.  At 60 experts with top-4 routing, 8 against 1:
    # batch 16 +2.3 %, 24 +5 %, 32 +6.4 %, 64 +3.5 %, 100 +9.7 %; at 9, 12 and 15 tokens (where 1 keeps the
    # mma.sync kernel) within 2 % either way.
    expert_skinny_rows_per_expert: int = 1

    # The shared expert runs on a second stream beside the routed experts: in decode-sized steps every
    # kernel is short, and in prefill its library products are bound by the tensor cores while the grouped
    # products of the routed experts are bound by memory (7 % off a 2,048-token prefill when introduced).
    shared_expert_overlap: bool = True
    # Steps above this size run the shared expert as library products whose blocks fill an SM; on a stream
    # of higher priority they take their SMs ahead of the routing's small kernels, which slip into what is
    # left, whatever order the two streams' first kernels reach the device in.
    shared_expert_priority_stream_min_tokens: int = 128
    # In the smallest steps the routing is a chain of short dependent loads that a concurrent weight
    # stream slows down, so there the shared expert is forked after the routing, not before it.
    shared_expert_fork_after_routing_max_tokens: int = 15
    # The same for larger decode steps, whose expert rows are sorted (routing and permutation in one launch):
    # up to this many tokens the shared expert's library products start after that launch, which they would
    # slow down, and run beside the routed products.  128 against 0 (always before): batch 16 +0.3 %,
    # 24 +1.5 %, 32 +1.1 %, 64 +2.5 %, 128 +0.4 %.  A prompt portion keeps the order "shared expert first":
    # its first library product is as long as routing, permutation and row gather together.
    shared_expert_fork_after_permutation_max_tokens: int = 128

    # Split-KV decode attention: keys per split by the number of requests in the step, as (up to this
    # many requests, keys per split) pairs, then the kernel's default of 512.  One or two requests alone
    # cannot fill 148 SMs with splits of 512 keys; splits of 256 for every batch size gained 4 % at batch 1
    # and lost 6 % at batch 8, hence the steps.  (bfloat16 path only: the float32 path runs one attention
    # kernel for every step, so that a request's logits do not depend on its batch.)
    decode_split_by_requests: Tuple[Tuple[int, int], ...] = ((2, 128), (4, 256))

    # Chunked prefill: every full portion of a long prompt has the same shape, so its forward pass is replayed
    # from a CUDA graph too, if a portion has at least this many tokens (0: never).  Below a few hundred
    # tokens a portion's kernels are too short for the saved launch gaps to matter against the memory a
    # captured pass holds.
    prefill_chunk_graph_min_tokens: int = 512

    # Steps of at most this many tokens ask L2 for the next dense weights (q/k/v, o_proj, shared expert)
    # on a second stream while a latency-bound kernel runs (0 = off).
    l2_prefetch_max_tokens: int = 15

    # Steps of at most this many tokens launch their kernels as programmatic dependents of the kernels before
    # them (0 = off): a kernel's blocks are placed while the one before it drains.  At A2.7B sizes: batch 1
    # +3.4 %, 2 +0.6 %, 4 +2.1 %, 8 +1.6 %; nothing either way from 16 tokens on, where library products stand
    # between the kernels that are written for it.  (Letting the next kernel's blocks in at a kernel's first
    # line instead of at its blocks' exit lost 5 to 8 % at batch 1 and 2: waiting blocks crowd the running ones.)
    dependent_launch_max_tokens: int = 15

    # Routing with the permutation as one launch (the last block builds the permutation) up to this many
    # tokens; above, logits kernel, selection kernel and permutation kernel (in isolation 18.5 against 30.8 us
    # at 128 tokens).  15 against 128, with the shared expert started after the routing: batch 16 +0.4 %,
    # 32 +1.1 %, 64 +0.2 %, 100 +0.2 %, 128 +1.0 %.
    route_with_permutation_one_launch_max_tokens: int = 15

    # A step with a prompt portion beside decoding requests serves the decoding requests (they stand first)
    # with the split-KV decode attention and the portion with the prefill attention, from this many decoding
    # requests on (below, two more launches per layer cost more than the prefill kernel's wasted tiles).
    mixed_step_decode_kernel_min_requests: int = 4

    # Decode steps are replayed from a pass captured per batch size.  Up to this size every batch size has its
    # own pass (the kernels of the smallest steps change with the size, and a request more means up to top_k
    # experts more to read: 9 requests run as 12 would take 5.1 instead of 4.2 ms); above it sizes are rounded
    # up to a multiple of 2 (to 32), 4 (to 64) or 8 and the step is filled up with rows of no request, which
    # costs a few per cent of a step at most and saves a capture (30-50 ms) per size that a batch passes
    # through while it grows and shrinks request by request.
    decode_graph_exact_batch_max: int = 16

    def decode_graph_batch(self, num_requests: int) -> int:
        if num_requests <= self.decode_graph_exact_batch_max:
            return num_requests
        step = 2 if num_requests <= 32 else (4 if num_requests <= 64 else 8)
        return -(-num_requests // step) * step

    def decode_split(self, num_requests: int, default: int) -> int:
        for limit, split in self.decode_split_by_requests:
            if num_requests <= limit:
                return split
        return default


def _from_environment(t: Tuning) -> Tuning:
    """``MINI_INFER_TUNING="name=value,name=value"`` overrides integer and boolean fields, for re-measuring a
    threshold without editing this file."""
    import os
    text = os.environ.get("MINI_INFER_TUNING", "")
    for item in filter(None, (x.strip() for x in text.split(","))):
        name, _, value = item.partition("=")
        if not hasattr(t, name) or isinstance(getattr(t, name), tuple):
            raise ValueError(f"MINI_INFER_TUNING: no integer or boolean threshold called '{name}'")
        old = getattr(t, name)
        setattr(t, name, (value.lower() in ("1", "true", "yes")) if isinstance(old, bool) else int(value))
    return t


TUNING = _from_environment(Tuning())
