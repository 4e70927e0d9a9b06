"""Multi-GPU use of the BitLinear path on one node: one process per GPU, torch.distributed for
the plumbing (NCCL on GPUs, gloo in CPU tests).

The reference has no distributed code (no NCCL/MPI anywhere in its sources); the two schemes
here are the ones the path shards into naturally:

* independent sequences (decode of many requests): token rows are split over ranks, weights
  are replicated, every rank runs the ordinary forward on its rows -- no collective at all;
* one oversized layer: the OUTPUT features are split.  Rank r owns rows
  [r*N/g, (r+1)*N/g) of W, which is a contiguous byte range of the canonical packed stream, computes
  y[:, slice] for all tokens, and the slices are all-gathered.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_range(n_items: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced [begin, end) of `n_items` for `rank` (sizes differ by at most one)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    return rank * n_items // world, (rank + 1) * n_items // world


def packed_row_slice(packed: torch.Tensor, out_features: int, in_features: int, world: int, rank: int):
    """This rank's rows of W as a view of the canonical packed stream, with its row range.

    The slice must start and end on a byte boundary of the flat 2-bit stream, i.e. row_begin*K and
    row_end*K must be multiples of 4 (always true when K % 4 == 0)."""
    r0, r1 = shard_range(out_features, world, rank)
    if (r0 * in_features) % 4 or (r1 * in_features) % 4:
        raise ValueError("row slice does not fall on a byte boundary of the packed stream")
    return packed.reshape(-1)[r0 * in_features // 4: r1 * in_features // 4], (r0, r1)


class NSplitBitLinear:
    """Output-feature-split BitLinear: local column slice, then an all-gather of the fp32 outputs.

    `compute(packed_slice, scale, x, n_local) -> y_local [M, n_local]` is the single-GPU forward
    (ops.bitlinear_forward on a GPU); it is a parameter so that the sharding and gathering logic
    can be exercised on CPU ranks."""

    def __init__(self, packed_full: torch.Tensor, scale: float, out_features: int, in_features: int,
                 compute: Callable | None = None, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if out_features % self.world:
            raise ValueError(f"out_features {out_features} must divide evenly over {self.world} ranks for the gather")
        self.out_features, self.in_features, self.scale = out_features, in_features, scale
        self.packed, (self.r0, self.r1) = packed_row_slice(packed_full, out_features, in_features, self.world, self.rank)
        self.packed = self.packed.contiguous()
        if compute is None:
            from . import ops
            compute = lambda wp, s, x, n: ops.bitlinear_forward(wp, s, x, n)   # noqa: E731
        self.compute = compute

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [M,K] (replicated on every rank) -> y [M,N] (complete on every rank)."""
        n_local = self.r1 - self.r0
        y_local = self.compute(self.packed, self.scale, x, n_local).contiguous()
        M = y_local.shape[0]
        gathered = torch.empty((self.world * M, n_local), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(gathered, y_local, group=self.group)   # rank r's slice lands in rows [r*M, (r+1)*M)
        return gathered.view(self.world, M, n_local).permute(1, 0, 2).reshape(M, self.out_features)


class FusedNSplitBitLinear:
    """Output-feature-split BitLinear without a collective: every rank's kernel (the decode kernel up to
    16 tokens, the persistent GEMM above) stores its column slice straight into ALL ranks' full-width
    outputs (plain peer stores over NVLink from the kernel's epilogue), and a symmetric-memory barrier
    tells the ranks that the slices have arrived.  The outputs live in torch symmetric memory, which maps every rank's
    buffer into every process.  Two output buffers alternate from call to call.  With `guard=True` (the default) a
    barrier before the launch keeps a fast rank from overwriting an output that a slow rank is still reading; with
    `guard=False` that barrier is dropped, which is safe when every rank is through with the result of call n before
    any rank passes the barrier of call n + 1 -- true for calls issued in stream order, one after the other, since a
    buffer is written again only by call n + 2 (a captured graph that holds ONE call replays the same buffer every
    time: keep the guard there)."""

    def __init__(self, packed_full: torch.Tensor, scale: float, out_features: int, in_features: int, max_tokens: int = 16,
                 group=None, share_outputs_with: "FusedNSplitBitLinear | None" = None):
        """share_outputs_with: another layer of the same output width, token limit and group whose two output buffers
        this one uses too (the layers of a model need one pair between them); the alternation then runs over the
        calls of all sharing layers."""
        import torch.distributed._symmetric_memory as symm_mem

        from . import ops
        self._ops = ops
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        self.out_features, self.in_features, self.scale, self.max_tokens = out_features, in_features, scale, max_tokens
        self.packed, (self.r0, self.r1) = packed_row_slice(packed_full, out_features, in_features, self.world, self.rank)
        self.packed = self.packed.contiguous()
        if (self.r0 * 4) % 16:
            raise ValueError("a rank's first column must be 16-byte aligned in the output row")
        if share_outputs_with is not None:
            o = share_outputs_with
            if (o.out_features, o.max_tokens, o.world) != (out_features, max_tokens, self.world):
                raise ValueError("layers that share outputs must agree on width, token limit and group size")
            self._out = o._out
        else:
            self._out = {"ys": [], "handles": [], "turn": 0}
            for _ in range(2):
                y = symm_mem.empty((max_tokens, out_features), dtype=torch.float32, device=packed_full.device)
                self._out["ys"].append(y)
                self._out["handles"].append(symm_mem.rendezvous(y, self.group))
        # this rank's slice inside every rank's output
        self.peer_ptrs = [[int(ptr) + 4 * self.r0 for ptr in h.buffer_ptrs] for h in self._out["handles"]]
        self._unused = torch.empty((max_tokens, self.r1 - self.r0), dtype=torch.float32, device=packed_full.device)

    def forward(self, x: torch.Tensor, guard: bool = True) -> torch.Tensor:
        """x [M,K] (replicated on every rank) -> y [M,N] (complete on every rank, a view of one of the two shared
        outputs; valid until the call after next)."""
        M = x.shape[0]
        if M > self.max_tokens:
            raise ValueError(f"{M} tokens > max_tokens {self.max_tokens}")
        t = self._out["turn"]
        self._out["turn"] = t ^ 1
        handle = self._out["handles"][t]
        if guard:
            handle.barrier(channel=0)   # nobody still reads what this buffer held
        self._ops.bitlinear_forward(self.packed, self.scale, x, self.r1 - self.r0, path="decode" if M <= 16 else "prefill",
                                    out=self._unused[:M], ldy=self.out_features, y_peers=self.peer_ptrs[t])
        handle.barrier(channel=1)   # every rank's slice has landed everywhere
        return self._out["ys"][t][:M]


def row_sharded_forward(forward: Callable[[torch.Tensor], torch.Tensor], x_all: torch.Tensor, group=None) -> torch.Tensor:
    """Independent token rows: this rank's share of `x_all` through `forward`; no communication.
    Returns the local outputs (callers that need all rows on one rank gather them themselves)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    b, e = shard_range(x_all.shape[0], world, rank)
    return forward(x_all[b:e].contiguous())
