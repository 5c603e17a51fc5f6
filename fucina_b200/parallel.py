"""Multi-GPU forms of the hot path: one process per GPU, torch.distributed for the exchange.

The reference is single-device (`cuDeviceGet(&c.device, 0)`, src/backend/cuda.zig:439); these are
the two exchange steps the path has when it is spread over NVLink-connected GPUs:

* `ColumnShardedLinear` -- tensor parallel by OUTPUT columns: rank r holds weight rows
  [r*N/G, (r+1)*N/G) (contiguous in the row-major block array, so sharding is a slice), the
  activations are replicated, every rank computes y_r = a . W_r^T and one all-gather assembles the
  result. No reduction is involved, so each output element is computed exactly as on one GPU.
* `ExpertParallelMoE` -- experts split E/G per rank, tokens sharded by rank, one all-to-all of the
  routed token rows to the ranks that own their experts, the expert FFN on the received rows, one
  all-to-all back, and the weighted sum in slot order on the token's home rank
  (src/exec/moe_chain.zig:307-330 keeps the same order).

Compute is injected (`gemm`, `expert_ffn` callables) so the sharding and exchange logic runs
unchanged on CPU tensors with the gloo backend in the tests and on CUDA tensors with NCCL in the
bench; collectives are issued on the current torch stream.
"""
from __future__ import annotations

from typing import Callable

import numpy as np
import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of an n-row matrix owned by `rank`: contiguous, multiples of 4 wide
    (the provider's n % 4 rule, src/backend/cuda.zig:2017), remainder spread over the first ranks."""
    if n % 4:
        raise ValueError("n must be a multiple of 4")
    q, r = divmod(n // 4, world)
    lo = 4 * (rank * q + min(rank, r))
    hi = lo + 4 * (q + (1 if rank < r else 0))
    return lo, hi


class ColumnShardedLinear:
    """y[m, N] = a[m, K] . dequant(W)^T with W's rows split over the ranks.

    `gemm(a) -> y_local [m, hi-lo]` computes this rank's columns (on the GPU: `fq_gemm_quant_nt_dev`
    on the rank's `Weights` shard). `forward` returns the gathered result as [world][m][cols]
    (rank-major; equal shards) or, for ragged shards, the concatenated [m, N].
    """

    def __init__(self, n: int, gemm: Callable[[torch.Tensor], torch.Tensor], group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n = n
        self.bounds = [shard_rows(n, self.world, r) for r in range(self.world)]
        self.lo, self.hi = self.bounds[self.rank]
        self.equal = len({hi - lo for lo, hi in self.bounds}) == 1
        self.gemm = gemm

    def forward(self, a: torch.Tensor) -> torch.Tensor:
        y_local = self.gemm(a)
        m = a.shape[0]
        assert y_local.shape == (m, self.hi - self.lo)
        if self.equal:
            out = torch.empty((self.world * m, self.hi - self.lo), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(out, y_local.contiguous(), group=self.group)
            return out.view(self.world, m, self.hi - self.lo)
        # ragged shards: gather at the widest shard's width, then drop the padding columns
        width = max(hi - lo for lo, hi in self.bounds)
        padded = torch.zeros((m, width), dtype=y_local.dtype, device=y_local.device)
        padded[:, : self.hi - self.lo] = y_local
        out = torch.empty((self.world * m, width), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(out, padded, group=self.group)
        out = out.view(self.world, m, width)
        return torch.cat([out[r, :, : hi - lo] for r, (lo, hi) in enumerate(self.bounds)], dim=1)

    @staticmethod
    def to_row_major(gathered: torch.Tensor) -> torch.Tensor:
        """[world][m][cols] -> [m][world*cols] (a view-changing copy; consumers that can index
        rank-major do not need it)."""
        if gathered.dim() == 2:
            return gathered
        w, m, c = gathered.shape
        return gathered.permute(1, 0, 2).reshape(m, w * c)


class ExpertParallelMoE:
    """Expert-parallel MoE layer over `world` ranks, `n_expert / world` consecutive experts each.

    `expert_ffn(x_rows [R, hidden], local_expert [R] int32) -> [R, hidden]` runs the gate/up/SwiGLU/
    down chain of one expert per row (on the GPU: `fq_moe_layer_dev` with top_k = 1 and weight 1).
    """

    def __init__(self, n_expert: int, top_k: int, expert_ffn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_expert % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.n_expert, self.top_k = n_expert, top_k
        self.per_rank = n_expert // self.world
        self.expert_ffn = expert_ffn

    def forward(self, x: torch.Tensor, selected: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """x [T_local, hidden] (this rank's tokens), selected/weights [T_local, top_k] -> [T_local, hidden]."""
        T, hidden = x.shape
        k = self.top_k
        sel = selected.reshape(-1).to(torch.int64)
        owner = sel // self.per_rank
        # stable sort of this rank's (token, slot) pairs by destination rank
        order = torch.sort(owner, stable=True).indices
        send_counts = torch.bincount(owner, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_list = send_counts.tolist()   # one host sync per layer: the exchange sizes
        recv_list = recv_counts.tolist()
        rows_out = x[order // k].contiguous()
        exp_out = (sel[order] % self.per_rank).to(torch.int32).contiguous()
        R = int(sum(recv_list))
        rows_in = torch.empty((R, hidden), dtype=x.dtype, device=x.device)
        exp_in = torch.empty((R,), dtype=torch.int32, device=x.device)
        dist.all_to_all_single(rows_in, rows_out, recv_list, send_list, group=self.group)
        dist.all_to_all_single(exp_in, exp_out, recv_list, send_list, group=self.group)
        y_in = self.expert_ffn(rows_in, exp_in) if R else rows_in
        y_back = torch.empty_like(rows_out)
        dist.all_to_all_single(y_back, y_in.contiguous(), send_list, recv_list, group=self.group)
        # y_back[i] belongs to pair order[i]; combine in slot order, first slot assigned
        pair_rows = torch.empty_like(y_back)
        pair_rows[order] = y_back
        pair_rows = pair_rows.view(T, k, hidden)
        w = weights.reshape(T, k).to(x.dtype)
        out = w[:, 0:1] * pair_rows[:, 0]
        for j in range(1, k):
            out = out + w[:, j:j + 1] * pair_rows[:, j]
        return out

    def forward_gathered(self, x: torch.Tensor, selected: torch.Tensor, weights: torch.Tensor,
                         partial_ffn: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                         chunks: int = 1, exchange_dtype=None) -> torch.Tensor:
        """The same layer with fixed-size exchanges and no host synchronisation: all-gather the token
        rows and their routing, let every rank compute the partial sums of ITS experts for all
        world*T tokens, and reduce-scatter the partial outputs back to the tokens' home ranks.

        `partial_ffn(x_all [W*T, hidden], selected_all [W*T, k] (global expert ids), weights_all)
        -> [W*T, hidden]` returns, per token, the slot-ordered weighted sum over the pairs this
        rank's experts serve and zero rows elsewhere (on the GPU: `fq_moe_layer_ep_dev`).

        Each token row crosses the links once per direction instead of once per routed pair, the
        sizes never depend on the routing, and NVSwitch can do the reduction in the fabric. A token's
        slots are summed per rank first and across ranks second, so the result differs from the
        single-GPU slot-order sum by f32 rounding (not bit-identical, unlike `forward`)."""
        T, hidden = x.shape
        k = self.top_k
        W = self.world
        # routing of every token, once. int32 ids and float32 weights have the same width, so they travel as one
        # [T, 2k] int32 tensor (one collective launch instead of two); other dtypes take two gathers.
        if selected.dtype == torch.int32 and weights.dtype == torch.float32:
            packed = torch.cat([selected.reshape(T, k), weights.reshape(T, k).view(torch.int32)], dim=1).contiguous()
            packed_all = torch.empty((W, T, 2 * k), dtype=torch.int32, device=x.device)
            dist.all_gather_into_tensor(packed_all.view(W * T, 2 * k), packed, group=self.group)
            sel_all = packed_all[:, :, :k]
            w_all = packed_all[:, :, k:].contiguous().view(torch.float32)
        else:
            sel_all = torch.empty((W, T, k), dtype=selected.dtype, device=x.device)
            w_all = torch.empty((W, T, k), dtype=weights.dtype, device=x.device)
            dist.all_gather_into_tensor(sel_all.view(W * T, k), selected.reshape(T, k).contiguous(), group=self.group)
            dist.all_gather_into_tensor(w_all.view(W * T, k), weights.reshape(T, k).contiguous(), group=self.group)
        out = torch.empty((T, hidden), dtype=x.dtype, device=x.device)
        gloo = dist.get_backend(self.group) == "gloo"   # gloo has no reduce-scatter: all-reduce and keep this rank's rows
        if chunks < 1 or T % chunks:
            chunks = 1
        # Token chunks pipeline the exchange against the expert products: while chunk c is multiplied, chunk c+1
        # is being gathered and chunk c-1 reduced (asynchronous collectives run on the communicator's own stream).
        h = T // chunks
        # token rows may cross the links in a narrower type (bf16 halves the gather; the tensor-core arm rounds
        # its activations to bf16 anyway, so prefill-sized batches lose nothing) and are widened again on arrival
        x_send = x.contiguous() if exchange_dtype is None else x.to(exchange_dtype).contiguous()
        gathers, xs = [], []
        for c in range(chunks):
            xc = torch.empty((W * h, hidden), dtype=x_send.dtype, device=x.device)
            gathers.append(dist.all_gather_into_tensor(xc, x_send[c * h:(c + 1) * h], group=self.group, async_op=not gloo))
            xs.append(xc)
        pending = []
        for c in range(chunks):
            if gathers[c] is not None:
                gathers[c].wait()
            # rows of chunk c in rank-major order, as the gather lays the tokens out
            sel_c = sel_all[:, c * h:(c + 1) * h].reshape(W * h, k)
            w_c = w_all[:, c * h:(c + 1) * h].reshape(W * h, k)
            partial = partial_ffn(xs[c] if exchange_dtype is None else xs[c].to(x.dtype), sel_c, w_c)
            if gloo:
                dist.all_reduce(partial, group=self.group)
                out[c * h:(c + 1) * h].copy_(partial[self.rank * h:(self.rank + 1) * h])
            else:
                pending.append((dist.reduce_scatter_tensor(out[c * h:(c + 1) * h], partial.contiguous(), group=self.group, async_op=True),
                                partial))
        for work, _keep_alive in pending:
            work.wait()
        return out

    def exchange_bytes(self, T: int, hidden: int, elem: int = 4) -> int:
        """Upper bound of bytes one rank sends per direction: every routed pair leaves the rank."""
        return T * self.top_k * hidden * elem


def numpy_to_torch(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a))
