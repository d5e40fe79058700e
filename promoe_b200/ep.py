"""Expert-parallel MoE layer over the ranks of one node (one process per GPU).

Tokens are data-parallel (every rank routes its own batch with a replicated router), routed
experts are sharded in contiguous blocks (`expert_bounds`), the shared expert is replicated.
Per layer there is one exchange each way:

    route + permute (rows sorted by expert = sorted by owner rank)
    -> all-to-all of the per-expert row counts
    -> all-to-all of the token rows                      (dispatch)
    -> owner: cache bookkeeping, copies, grouped FFN     (pm_moe_forward_routed, own expert cache)
    -> all-to-all of the expert outputs, f32             (combine traffic)
    -> source: weighted combine + shared expert

The reference has no multi-GPU path (device 0 is hard-coded, src/cpp_worker/model_loader.cpp:75-79),
so there is nothing to mirror: each rank's cache behaves exactly like a single-GPU cache over its
block of experts, fed with the union of the ids that arrive from all ranks.

Collectives go through torch.distributed (NCCL over NVLink for CUDA tensors, gloo for the CPU
tests); all device compute goes through the C ABI via a small backend object, so the host logic
(bucketing, split sizes, round trip) can be exercised without a GPU by passing another backend.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist


def expert_bounds(num_expert: int, world: int) -> list[int]:
    """Block boundaries: rank r owns experts [bounds[r], bounds[r+1])."""
    return [r * num_expert // world for r in range(world + 1)]


def split_counts(counts: torch.Tensor, bounds: list[int]) -> list[int]:
    """Rows per destination rank from the per-expert row counts (host tensor)."""
    return [int(counts[bounds[r]:bounds[r + 1]].sum()) for r in range(len(bounds) - 1)]


class CudaBackend:
    """Device work of one rank through the C ABI (stateless kernels + the rank's ExpertCache)."""

    def __init__(self, cache, layers, device):
        """layers[l] = dict(gate_w, gate_bias, shared (3 tensors or None), shared_gate_w, top_k, norm_topk,
        routed_scale, inter) with full-width (all experts) router weights."""
        from . import _lib
        self._lib, self.cache, self.layers, self.device = _lib, cache, layers, torch.device(device)
        self._scratch = None

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def route(self, layer, x):
        p, (T, H) = self.layers[layer], x.shape
        E, k = p["gate_w"].shape[0], p["top_k"]
        ids = torch.empty((T, k), dtype=torch.int32, device=self.device)
        w = torch.empty((T, k), dtype=torch.float32, device=self.device)
        ss = torch.empty((T,), dtype=torch.float32, device=self.device) if p["shared_gate_w"] is not None else None
        ptr = lambda t: None if t is None else t.data_ptr()  # noqa: E731
        self._lib.call("pm_k_gate_topk", x.data_ptr(), p["gate_w"].data_ptr(), ptr(p["gate_bias"]),
                       ptr(p["shared_gate_w"]), T, H, E, k, int(p["norm_topk"]), float(p["routed_scale"]), None,
                       ids.data_ptr(), w.data_ptr(), None, ptr(ss), None, self._stream())
        return ids, w, ss

    def permute(self, ids, num_expert):
        T, k = ids.shape
        R = T * k
        counts = torch.empty(num_expert, dtype=torch.int32, device=self.device)
        offsets = torch.empty(num_expert + 1, dtype=torch.int32, device=self.device)
        row_token = torch.empty(max(R, 1), dtype=torch.int32, device=self.device)
        pos = torch.empty(max(R, 1), dtype=torch.int32, device=self.device)
        self._lib.call("pm_k_permute", ids.data_ptr(), R, k, num_expert, counts.data_ptr(), offsets.data_ptr(),
                       row_token.data_ptr(), pos.data_ptr(), None, self._stream())
        return counts, offsets, row_token[:R], pos[:R]

    def gather_rows(self, src, index):
        out = torch.empty((index.shape[0], src.shape[1]), dtype=src.dtype, device=self.device)
        if index.shape[0]:
            self._lib.call("pm_k_gather_rows", src.data_ptr(), index.data_ptr(), index.shape[0],
                           src.shape[1] * src.element_size(), out.data_ptr(), self._stream())
        return out

    def expert_rows(self, layer, x_rows, row_expert):
        """Unweighted expert output (f32) of every received row, in arrival order."""
        out = torch.empty((x_rows.shape[0], x_rows.shape[1]), dtype=torch.float32, device=self.device)
        if x_rows.shape[0]:
            self._lib.call("pm_moe_forward_routed", self.cache.handle, layer, x_rows.data_ptr(), x_rows.shape[0],
                           row_expert.data_ptr(), out.data_ptr(), self._stream())
        return out

    def shared_rows(self, layer, x, yexp, first_row):
        """Writes the shared expert's output of every token into yexp[first_row : first_row + T]."""
        p = self.layers[layer]
        if p["shared"] is None:
            return
        T, H = x.shape
        sg, su, sd = p["shared"]
        inter = sg.shape[0]
        n_rows = first_row + T
        g = (self._lib.pm_ffn_group * 1)()
        g[0] = self._lib.pm_ffn_group(sg.data_ptr(), su.data_ptr(), sd.data_ptr(), None, None, None, first_row, T, inter, 0)
        row_token = torch.zeros(n_rows, dtype=torch.int32, device=self.device)
        row_token[first_row:] = torch.arange(T, dtype=torch.int32, device=self.device)
        nbytes = self._lib.call("pm_k_swiglu_ffn_scratch_bytes", 1, n_rows, inter, H)
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._lib.call("pm_k_swiglu_ffn", g, 1, 0, x.data_ptr(), H, row_token.data_ptr(), n_rows, yexp.data_ptr(),
                       self._scratch.data_ptr(), self._scratch.numel(), self._stream())

    def combine(self, yexp, pos, w, T, H, n_routed_rows, n_shared, shared_scale):
        y = torch.empty((T, H), dtype=torch.bfloat16, device=self.device)
        self._lib.call("pm_k_combine", yexp.data_ptr(), pos.data_ptr(), w.data_ptr(), T, H, w.shape[1], n_routed_rows,
                       n_shared, None if shared_scale is None else shared_scale.data_ptr(), y.data_ptr(), self._stream())
        return y


class ExpertParallelMoE:
    """The exchange logic of one rank. `backend` does the arithmetic (CudaBackend in production)."""

    def __init__(self, num_expert: int, backend, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.num_expert = num_expert
        self.bounds = expert_bounds(num_expert, self.world)
        self.max_block = max(self.bounds[r + 1] - self.bounds[r] for r in range(self.world))
        self.backend = backend
        self.bytes_dispatched = 0
        self.bytes_returned = 0

    def forward(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        be, G = self.backend, self.world
        T, H = x.shape
        ids, w, shared_scale = be.route(layer, x)
        k = ids.shape[1]
        R = T * k
        counts, offsets, row_token, pos = be.permute(ids, self.num_expert)
        x_sorted = be.gather_rows(x, row_token)  # rows sorted by expert id = grouped by owner rank

        # per-expert counts to the owners: a [G, max_block] table each way
        send_tab = torch.zeros((G, self.max_block), dtype=torch.int32, device=x.device)
        for r in range(G):
            send_tab[r, : self.bounds[r + 1] - self.bounds[r]] = counts[self.bounds[r]:self.bounds[r + 1]]
        recv_tab = torch.empty_like(send_tab)
        if G > 1:
            dist.all_to_all_single(recv_tab, send_tab, group=self.group)
        else:
            recv_tab.copy_(send_tab)
        send_rows = send_tab.sum(dim=1).tolist()      # host sync: split sizes must be known
        recv_tab_h = recv_tab.cpu()
        recv_rows = recv_tab_h.sum(dim=1).tolist()

        x_recv = torch.empty((sum(recv_rows), H), dtype=x.dtype, device=x.device)
        if G > 1:
            dist.all_to_all_single(x_recv, x_sorted, output_split_sizes=recv_rows, input_split_sizes=send_rows,
                                   group=self.group)
        else:
            x_recv.copy_(x_sorted)
        self.bytes_dispatched += x_sorted.numel() * x_sorted.element_size()

        n_local = self.bounds[self.rank + 1] - self.bounds[self.rank]
        local_ids = torch.arange(n_local, dtype=torch.int32).repeat(G)
        row_expert = torch.repeat_interleave(local_ids, recv_tab_h[:, :n_local].reshape(-1).long()).to(x.device)
        y_recv = be.expert_rows(layer, x_recv, row_expert)  # f32 [rows received, H], arrival order

        yexp = torch.empty((R + T, H), dtype=torch.float32, device=x.device)  # routed rows, then shared rows
        if G > 1:
            dist.all_to_all_single(yexp[:R], y_recv, output_split_sizes=send_rows, input_split_sizes=recv_rows,
                                   group=self.group)
        else:
            yexp[:R].copy_(y_recv)
        self.bytes_returned += y_recv.numel() * 4
        has_shared = be.layers[layer]["shared"] is not None
        if has_shared:
            be.shared_rows(layer, x, yexp, R)
        return be.combine(yexp, pos, w, T, H, R, 1 if has_shared else 0, shared_scale)
