"""Expert-parallel MoE layer over the ranks of one node (one process per GPU).

Tokens are data-parallel (every rank routes its own batch with a replicated router), routed
experts are sharded in contiguous blocks (`expert_bounds`), the shared expert is replicated.
Per layer there is ONE collective each way, with split sizes fixed in advance:

    route + permute + predictor scores of this rank's tokens      (source)
    pack: one fixed-size message per owner = header row (per-expert row counts, predictor scores
          of the owner's experts) + the token rows routed to the owner's experts
    -> all-to-all                                                 (dispatch)
    owner: unpack the headers into a row list (padding rows = -1), sum the predictor scores of all
           experts over the sources (every owner gets the same sums, hence the same global ranking),
           pm_moe_forward_routed: prefetch those of the globally best-ranked experts that it owns,
           cache bookkeeping, copies, grouped FFN; the one host <-> device sync of the layer is its
           read of the row counts
    -> all-to-all of the expert outputs (f32, same geometry)      (combine traffic)
    source: shared expert (on a side stream, under the exchange) + weighted combine

The reference has no multi-GPU path (device 0 is hard-coded, src/cpp_worker/model_loader.cpp:75-79),
so there is nothing to mirror: each rank's cache behaves exactly like a single-GPU cache over its
block of experts, fed with the union of the ids that arrive from all ranks; and all ranks together
prefetch exactly the experts a single cache over all experts would: the top n of the predictor
scores summed over all ranks' tokens, each prefetched by its owner.

Collectives go through torch.distributed (NCCL over NVLink for CUDA tensors, gloo for the CPU
tests); all device compute goes through the C ABI via a backend object, so the host logic
(message geometry, reply positions, score sums) can be exercised without a GPU by passing a
backend that restates the kernels in numpy.
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


class Geometry:
    """Message geometry, identical on every rank: `cap` = most rows one source can send one owner
    (its tokens times top_k), a message is 1 header row + cap rows of `hidden` elements."""

    def __init__(self, num_expert: int, world: int, max_tokens_per_rank: int, top_k: int, hidden: int, n_pred: int = 0):
        self.num_expert, self.world, self.top_k, self.hidden, self.n_pred = num_expert, world, top_k, hidden, n_pred
        self.bounds = expert_bounds(num_expert, world)
        self.max_block = max(self.bounds[r + 1] - self.bounds[r] for r in range(world))
        self.cap = max_tokens_per_rank * top_k
        self.seg_rows = 1 + self.cap
        self.rows = world * self.seg_rows
        if (self.max_block + n_pred * num_expert) * 4 > hidden * 2:
            raise ValueError("the message header (counts and predictor scores) does not fit one row")


class CudaBackend:
    """Device work of one rank through the C ABI (stateless kernels + the rank's ExpertCache)."""

    def __init__(self, cache, layers, device, geometry: Geometry, rank: int, predictors=None, predict_map=None,
                 global_tokens: int = 0, n_predict: int = 0):
        """layers[l] = dict(gate_w, gate_bias, shared (3 tensors or None), shared_gate_w, top_k, norm_topk,
        routed_scale, inter) with full-width (all experts) router weights. predictors[(src, dst)] =
        (w1, b1, w2, b2) device tensors over ALL experts; predict_map[src] = (first, last + 1) of the
        layers index src predicts; n_predict: experts prefetched per predicted layer over ALL ranks
        (the global top n_predict; every owner prefetches the ones it holds). global_tokens: tokens in
        flight on all ranks per layer call (the bound on the rows one expert can receive), 0 if unknown."""
        from . import _lib
        self._lib, self.cache, self.layers, self.device = _lib, cache, layers, torch.device(device)
        self.geo, self.rank = geometry, rank
        self.n_local = geometry.bounds[rank + 1] - geometry.bounds[rank]
        self.predictors, self.predict_map = predictors or {}, predict_map
        self.global_tokens, self.n_predict = global_tokens, n_predict
        g, dev = geometry, self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.bounds_dev = torch.tensor(g.bounds, **i32)
        self.send = torch.zeros((g.rows, g.hidden), dtype=torch.bfloat16, device=dev)
        self.recv = torch.zeros_like(self.send)
        self.out = torch.zeros((g.rows, g.hidden), dtype=torch.float32, device=dev)
        self.row_expert = torch.empty(g.rows, **i32)
        self.unpack_err = torch.zeros(1, **i32)
        self.scores = torch.zeros((max(1, g.n_pred), g.num_expert), dtype=torch.float32, device=dev)
        self.scores_sum = torch.zeros((max(1, g.n_pred), g.num_expert), dtype=torch.float32, device=dev)
        self.pred_hidden = None
        self._per_tokens = {}
        self.side = torch.cuda.Stream(device=dev)
        self._shared_scratch = None
        self.launches = 0   # kernels this backend launched itself (the cache counts its own)
        self.pool = None    # set by enable_pool

    def enable_pool(self, arena_prefixes, n_local_of, mailbox_name: str, group=None, max_misses: int = 48):
        """Pooled miss fetch: every rank pulls 1/world of each missing expert record over its own host
        link and the slices meet at the owner over NVLink (see include/promoe_b200.h). The cache must
        have been pinned with the context option shared_arena = arena_prefixes[rank]; every rank calls
        this at the same point (it contains barriers)."""
        world, rank, h = self.geo.world, self.rank, self.cache.handle
        self._lib.call("pm_pool_init", h, rank, world, mailbox_name.encode())
        if world > 1:
            dist.barrier(group=group)      # every arena exists and is filled
            for peer in range(world):
                if peer != rank:
                    self._lib.call("pm_pool_open_peer", h, peer, arena_prefixes[peer].encode(), int(n_local_of[peer]))
            dist.barrier(group=group)
        slice_bytes = int(self.cache.get("pool_slice"))
        cap = max_misses * slice_bytes
        self.pool = dict(seq=0, cap=cap, max_misses=max_misses, slice=slice_bytes, group=group,
                         send=torch.empty(cap, dtype=torch.uint8, device=self.device),
                         recv=torch.empty(cap, dtype=torch.uint8, device=self.device),
                         stream=torch.cuda.Stream(device=self.device),
                         miss=(C.c_int32 * 64)(), lists=(C.c_int32 * (world * 65))(),
                         send_split=(C.c_int64 * world)(), recv_split=(C.c_int64 * world)(),
                         exchanges=0, local_fallbacks=0)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def buffers(self, T: int) -> dict:
        """Everything whose size depends on the number of local tokens, allocated once per size."""
        b = self._per_tokens.get(T)
        if b is not None:
            return b
        g, dev = self.geo, self.device
        k, E, H = g.top_k, g.num_expert, g.hidden
        R = T * k
        i32 = dict(dtype=torch.int32, device=dev)
        max_slices = 8
        b = dict(ids=torch.empty((T, k), **i32), w=torch.empty((T, k), dtype=torch.float32, device=dev),
                 ss=torch.empty((T,), dtype=torch.float32, device=dev), counts=torch.empty(E, **i32),
                 offsets=torch.empty(E + 1, **i32), row_token=torch.empty(max(R, 1), **i32),
                 pos=torch.empty(max(R, 1), **i32), pos_reply=torch.empty(max(R, 1), **i32),
                 reply=torch.zeros((g.rows + max_slices * T, H), dtype=torch.float32, device=dev),
                 y=torch.empty((T, H), dtype=torch.bfloat16, device=dev))
        # row table of the shared expert's launch: yexp row g.rows + j * T + t reads token t
        rt = torch.zeros(g.rows + max_slices * T, **i32)
        rt[g.rows:] = torch.arange(T, **i32).repeat(max_slices)
        b["shared_row_token"] = rt
        self._per_tokens[T] = b
        return b

    def route(self, layer, x, b):
        p, (T, H) = self.layers[layer], x.shape
        E, k = p["gate_w"].shape[0], p["top_k"]
        ptr = lambda t: None if t is None else t.data_ptr()  # noqa: E731
        has_gate = p["shared_gate_w"] is not None
        self._lib.call("pm_k_gate_topk", x.data_ptr(), p["gate_w"].data_ptr(), ptr(p["gate_bias"]),
                       ptr(p["shared_gate_w"]), T, H, E, k, int(p["norm_topk"]), float(p["routed_scale"]), None,
                       b["ids"].data_ptr(), b["w"].data_ptr(), None, b["ss"].data_ptr() if has_gate else None, None,
                       self._stream())
        self.launches += 1
        return b["ids"], b["w"], b["ss"] if has_gate else None

    def permute(self, ids, b):
        T, k = ids.shape
        self._lib.call("pm_k_permute", ids.data_ptr(), T * k, k, self.geo.num_expert, b["counts"].data_ptr(),
                       b["offsets"].data_ptr(), b["row_token"].data_ptr(), b["pos"].data_ptr(), None, self._stream())
        self.launches += 1
        return b["counts"], b["offsets"], b["row_token"], b["pos"]

    def predict(self, layer, x):
        """Predictor scores of this rank's tokens for the layers index `layer` predicts:
        (scores [n, num_expert] device f32 or None, [dst layers])."""
        if not self.predictors or self.predict_map is None:
            return None, []
        dsts = [d for d in range(*self.predict_map[layer]) if (layer, d) in self.predictors][: self.geo.n_pred]
        T, H = x.shape
        for i, d in enumerate(dsts):
            w1, b1, w2, b2 = self.predictors[(layer, d)]
            if self.pred_hidden is None or self.pred_hidden.numel() < T * w1.shape[0]:
                self.pred_hidden = torch.empty(T * w1.shape[0], dtype=torch.float32, device=self.device)
            self._lib.call("pm_k_predictor_mlp", x.data_ptr(), T, H, w1.data_ptr(),
                           None if b1 is None else b1.data_ptr(), w1.shape[0], w2.data_ptr(),
                           None if b2 is None else b2.data_ptr(), self.geo.num_expert, self.pred_hidden.data_ptr(),
                           self.scores[i].data_ptr(), self._stream())
            self.launches += 2
        return (self.scores if dsts else None), dsts

    def pack(self, x, b, scores, n_pred):
        g = self.geo
        T = x.shape[0]
        self._lib.call("pm_k_ep_pack", x.data_ptr(), g.hidden, b["counts"].data_ptr(), b["offsets"].data_ptr(),
                       b["row_token"].data_ptr(), b["pos"].data_ptr(), T * g.top_k, self.bounds_dev.data_ptr(), g.world,
                       g.max_block, g.cap, None if scores is None else scores.data_ptr(), n_pred, g.num_expert,
                       self.send.data_ptr(), b["pos_reply"].data_ptr(), self._stream())
        self.launches += 1
        return self.send, b["pos_reply"]

    def unpack(self, recv, n_pred):
        g = self.geo
        self._lib.call("pm_k_ep_unpack", recv.data_ptr(), g.hidden, g.world, self.n_local, g.max_block, g.cap, n_pred,
                       g.num_expert, self.row_expert.data_ptr(), self.scores_sum.data_ptr(), self.unpack_err.data_ptr(), self._stream())
        self.launches += 1
        return self.row_expert, (self.scores_sum if n_pred else None)

    def expert_rows(self, layer, recv, row_expert, scores_sum, dsts):
        """Unweighted expert output (f32) of every received row, in place of the row (padding -> zeros)."""
        arr = (C.c_int32 * max(1, len(dsts)))(*dsts)
        pred = (None if scores_sum is None else scores_sum.data_ptr(), arr, len(dsts), self.geo.num_expert,
                self.geo.bounds[self.rank], self.n_predict)
        if self.pool is None:
            self._lib.call("pm_moe_forward_routed", self.cache.handle, layer, recv.data_ptr(), self.geo.rows,
                           row_expert.data_ptr(), self.out.data_ptr(), self.global_tokens, *pred, self._stream())
            return self.out
        p, h, world = self.pool, self.cache.handle, self.geo.world
        n = C.c_int(0)
        self._lib.call("pm_moe_forward_routed_begin", h, layer, recv.data_ptr(), self.geo.rows, row_expert.data_ptr(),
                       self.out.data_ptr(), self.global_tokens, *pred, self._stream(), p["miss"],
                       min(64, p["max_misses"]), C.byref(n))
        p["seq"] += 1
        self._lib.call("pm_pool_exchange", h, p["seq"], p["miss"], n.value, p["lists"], 20.0)
        total = sum(p["lists"][r * 65] for r in range(world))
        if total > p["max_misses"]:          # every rank sees the same lists and takes the same branch
            self._lib.call("pm_pool_fetch_locally", h)
            p["local_fallbacks"] += 1
        elif total > 0:
            ps = p["stream"]
            with torch.cuda.stream(ps):
                self._lib.call("pm_pool_stage", h, layer, p["lists"], p["send"].data_ptr(), p["cap"], p["cap"],
                               p["send_split"], p["recv_split"], ps.cuda_stream)
                ins, outs = list(p["send_split"]), list(p["recv_split"])
                if world > 1:
                    dist.all_to_all_single(p["recv"][: sum(outs)], p["send"][: sum(ins)], outs, ins, group=p["group"])
                else:
                    p["recv"][: sum(outs)].copy_(p["send"][: sum(ins)])
                self._lib.call("pm_pool_scatter", h, p["recv"].data_ptr(), ps.cuda_stream)
            p["exchanges"] += 1
        self._lib.call("pm_moe_forward_routed_end", h)
        return self.out

    def shared_begin(self, layer, x, b):
        """Launches the shared expert of every local token on a side stream; its rows land behind the
        reply rows of b['reply'] (one block of T rows per slice of the intermediate dimension)."""
        p = self.layers[layer]
        if p["shared"] is None:
            return 0
        T, H = x.shape
        sg, su, sd = p["shared"]
        inter_sh, inter = sg.shape[0], p["inter"]
        # same slicing as the single-GPU layer: about one routed expert's width per slice, at most 8
        width = max(inter, -(-inter_sh // 8))
        width = min(-(-width // 32) * 32, inter_sh)
        n_slices = -(-inter_sh // width) if T <= 16 else 1
        if n_slices == 1:
            width = inter_sh
        first = self.geo.rows
        groups = (self._lib.pm_ffn_group * n_slices)()
        for j in range(n_slices):
            wj = min(width, inter_sh - j * width)
            groups[j] = self._lib.pm_ffn_group(sg.data_ptr() + j * width * H * 2, su.data_ptr() + j * width * H * 2,
                                               sd.data_ptr() + j * width * 2, None, None, None, first + j * T, T, wj,
                                               inter_sh)
        n_rows = first + n_slices * T
        nbytes = self._lib.call("pm_k_swiglu_ffn_scratch_bytes", n_slices, n_rows, width, H)
        if self._shared_scratch is None or self._shared_scratch.numel() < nbytes:
            self._shared_scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.side):
            self._lib.call("pm_k_swiglu_ffn", groups, n_slices, 0, x.data_ptr(), H, b["shared_row_token"].data_ptr(),
                           n_rows, b["reply"].data_ptr(), self._shared_scratch.data_ptr(),
                           self._shared_scratch.numel(), self.side.cuda_stream)
        self.launches += 1
        return n_slices

    def shared_end(self):
        torch.cuda.current_stream(self.device).wait_stream(self.side)

    def combine(self, b, pos_reply, w, T, n_shared, shared_scale):
        g = self.geo
        self._lib.call("pm_k_combine", b["reply"].data_ptr(), pos_reply.data_ptr(), w.data_ptr(), T, g.hidden, g.top_k,
                       g.rows, n_shared, None if shared_scale is None else shared_scale.data_ptr(), b["y"].data_ptr(),
                       self._stream())
        self.launches += 1
        return b["y"]


class ExpertParallelMoE:
    """The exchange logic of one rank. `backend` does the arithmetic (CudaBackend in production)."""

    def __init__(self, geometry: Geometry, backend, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if geometry.world != self.world:
            raise ValueError("the message geometry was built for another world size")
        self.geo, self.backend = geometry, backend
        self.bytes_dispatched = 0
        self.bytes_returned = 0
        self.trace = None   # set to a list to record CUDA events at the phase boundaries of every layer call

    def _mark(self, marks):
        if self.trace is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append(e)

    def trace_summary(self) -> dict:
        """Mean microseconds per layer call of each phase, from the recorded events (after a synchronize)."""
        names = ("route_permute_pack", "dispatch_all_to_all", "owner_unpack_ffn_copies", "reply_all_to_all", "combine")
        tot = dict.fromkeys(names, 0.0)
        for marks in self.trace:
            for i, n in enumerate(names):
                tot[n] += marks[i].elapsed_time(marks[i + 1]) * 1e3
        n_calls = max(1, len(self.trace))
        return {k: v / n_calls for k, v in tot.items()}

    def _exchange(self, dst: torch.Tensor, src: torch.Tensor):
        """Equal-split all-to-all of two buffers of the same geometry, as bytes."""
        if self.world > 1:
            dist.all_to_all_single(dst.view(torch.uint8).view(-1), src.view(torch.uint8).view(-1), group=self.group)
        else:
            dst.copy_(src)

    def forward(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        be, g = self.backend, self.geo
        T = x.shape[0]
        if T * g.top_k > g.cap:
            raise ValueError(f"{T} tokens exceed the message capacity ({g.cap} rows per peer)")
        b = be.buffers(T)
        marks = []
        self._mark(marks)
        ids, w, shared_scale = be.route(layer, x, b)
        be.permute(ids, b)
        scores, dsts = be.predict(layer, x)
        n_shared = be.shared_begin(layer, x, b)           # runs under the exchange
        send, pos_reply = be.pack(x, b, scores, len(dsts))
        self._mark(marks)
        self._exchange(be.recv, send)                     # dispatch
        self.bytes_dispatched += send.numel() * send.element_size()
        self._mark(marks)
        row_expert, scores_sum = be.unpack(be.recv, len(dsts))
        out = be.expert_rows(layer, be.recv, row_expert, scores_sum, dsts)
        self._mark(marks)
        self._exchange(b["reply"][: g.rows], out)          # expert outputs back to their sources
        self.bytes_returned += out.numel() * out.element_size()
        self._mark(marks)
        if n_shared:
            be.shared_end()
        y = be.combine(b, pos_reply, w, T, n_shared, shared_scale)
        self._mark(marks)
        if self.trace is not None:
            self.trace.append(marks)
        return y
