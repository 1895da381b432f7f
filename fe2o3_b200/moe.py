"""MoE top-2 layer: gate -> top-2 routing -> route weights -> expert FFN -> combine.

Single GPU: the host schedule of examples/moe_expert_v1/src/pipeline.rs:166-270
(compact accepted routes by expert, run the experts, inverse-permute, combine in
rank order) with every stage a launch through the C ABI.

Several GPUs (one process per GPU, `torch.distributed`): tokens are split
across ranks and experts are block-partitioned.  Each rank routes its own
tokens; rows bound for experts on other ranks travel in one all-to-all
(dispatch), the owning rank runs the grouped FFN, and a second all-to-all
(combine) brings the rows back to the token's home rank, where the weighted
combine runs in rank order.  torch is used for device memory and NCCL plumbing
only; every arithmetic stage is a kernel of libfe2o3_b200.so.
"""
import numpy as np

from . import SCHEDULE_AUTO, prepare  # noqa: F401

DROP = 0xFFFFFFFF


def split_plan(counts, rank, world):
    """Pure host logic of the exchange, from the gathered per-(source rank,
    expert) route counts `counts[world][experts]`.

    Returns (send_rows, recv_rows, group_offsets): rows this rank sends to each
    destination, rows it receives from each source, and the exclusive scan of
    the received segments in arrival order (source-major, local expert minor),
    which is the row partition of the grouped FFN."""
    counts = np.asarray(counts, np.int64)
    experts = counts.shape[1]
    per = experts // world
    send_rows = [int(counts[rank, d * per:(d + 1) * per].sum()) for d in range(world)]
    recv_seg = counts[:, rank * per:(rank + 1) * per]  # [source][local expert]
    recv_rows = [int(recv_seg[s].sum()) for s in range(world)]
    group_offsets = np.zeros(world * per + 1, np.uint32)
    group_offsets[1:] = np.cumsum(recv_seg.reshape(-1))
    return send_rows, recv_rows, group_offsets


class MoeTop2Layer:
    def __init__(self, ctx, stream, tokens, d_model, d_ff, experts, rank=0, world=1, capacity=None, exchange="auto"):
        import torch
        self.torch = torch
        self.exchange = "none" if world == 1 else exchange
        assert experts % world == 0 and tokens % world == 0
        self.ctx, self.stream = ctx, stream
        self.rank, self.world = rank, world
        self.T, self.d, self.f, self.E = tokens // world, d_model, d_ff, experts
        self.per = experts // world
        self.R = 2 * self.T
        self.capacity = self.R if capacity is None else capacity
        dev = torch.device("cuda", torch.cuda.current_device())
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)
        T, d, f, E, R = self.T, d_model, d_ff, experts, self.R
        self.x = z(T * d, torch.bfloat16)
        self.wg = z(d * E, torch.bfloat16)
        self.w1 = z(self.per * d * f, torch.bfloat16)   # this rank's experts only
        self.w2 = z(self.per * f * d, torch.bfloat16)
        self.logits = z(T * E, torch.float32)
        self.top2, self.slots, self.perm, self.inverse = (z(R, torch.int32) for _ in range(4))
        self.requested, self.admitted = z(E, torch.int32), z(E, torch.int32)
        self.offsets = z(E + 1, torch.int32)
        self.weights = z(R, torch.float32)
        self.out = z(T * d, torch.float32)
        # rows this rank may have to process: every route of every rank in the worst case
        self.max_rows = R * world
        self.compact_x = z(R * d, torch.bfloat16)            # local routes, expert-major
        self.compact_out = z(R * d, torch.float32)           # FFN rows back in local slot order
        if world > 1 and self.exchange in ("auto", "peer"):
            try:
                self._setup_peer_buffers(dev)
                self.exchange = "peer"
            except Exception as err:  # symmetric memory unavailable: use the NCCL all-to-all path
                if self.exchange == "peer":
                    raise
                self.exchange, self.exchange_fallback_reason = "nccl", f"{type(err).__name__}: {err}"
        if world > 1:
            if self.exchange == "nccl":
                self.recv_x = z(self.max_rows * d, torch.bfloat16)
                self.ffn_out = z(self.max_rows * d, torch.float32)
            self.group_offsets = z(E + 1, torch.int32)
            self.counts_all = z(world * E, torch.int32)
            self.host_counts = torch.zeros(world * E, dtype=torch.int32).pin_memory()
            self.host_group_offsets = torch.zeros(E + 1, dtype=torch.int32).pin_memory()
            rows, ffn_in, ffn_res, ffn_off = self.max_rows, self.recv_x, self.ffn_out, self.group_offsets
        else:
            rows, ffn_in, ffn_res, ffn_off = R, self.compact_x, self.compact_out, self.offsets
        self.hidden = z(rows * f, torch.bfloat16)
        self.rows = rows
        P = lambda op, **kw: prepare(ctx, op, **kw)
        self.k_gate = P("moe_gate_v1", x=self.x, wg=self.wg, logits=self.logits, tokens=T, d_model=d, experts=E)
        self.k_top2 = P("moe_top2_v1", logits=self.logits, top2_experts=self.top2, requested_counts=self.requested,
                        admitted_counts=self.admitted, expert_offsets=self.offsets, route_slots=self.slots,
                        permutation=self.perm, inverse=self.inverse, tokens=T, experts=E, capacity=self.capacity)
        self.k_weights = P("moe_route_weights_v1", logits=self.logits, top2_experts=self.top2,
                           route_weights=self.weights, tokens=T, experts=E)
        if world == 1:
            self.k_ffn = P("moe_expert_ffn_v1", x=self.x, w1=self.w1, w2=self.w2, permutation=self.perm,
                           expert_offsets=self.offsets, compact_x=self.compact_x, hidden=self.hidden,
                           compact_output=self.compact_out, tokens=T, d_model=d, d_ff=f, experts=E)
        else:
            self.k_compact = P("moe_compact_v1", x=self.x, permutation=self.perm, compact_x=self.compact_x,
                               tokens=T, d_model=d)
            self.k_ffn = P("moe_grouped_ffn_v1", compact_x=ffn_in, w1=self.w1, w2=self.w2, group_offsets=ffn_off,
                           hidden=self.hidden, compact_output=ffn_res, d_model=d, d_ff=f, groups=E,
                           experts_cycle=self.per)
        self.k_combine = P("moe_expert_combine_v1", compact_output=self.compact_out, inverse=self.inverse,
                           route_weights=self.weights, combined_output=self.out, tokens=T, width=d)
        if self.exchange == "peer":
            from ._lib import MoeEpExchangeArgs
            self.remote_rows = z(R, torch.int32)
            self.epoch_counter = z(1, torch.int32)  # pass number, advanced on the device: passes replay from a graph
            self.k_phase = [P("moe_ep_exchange_v1", x=self.x, top2_experts=self.top2, permutation=self.perm,
                              inverse=self.inverse, expert_offsets=self.offsets, requested_counts=self.requested,
                              route_weights=self.weights, group_offsets=self.group_offsets,
                              remote_rows=self.remote_rows, combined_output=self.out, peer_recv_x=self.peer_recv_x,
                              peer_ffn_out=self.peer_ffn_out, peer_counts=self.peer_counts,
                              peer_flags=self.peer_flags, epoch_counter=self.epoch_counter, tokens=T, d_model=d,
                              experts=E, world=world, rank=rank, epoch=0, max_rows=self.max_rows, phase=ph)
                            for ph in range(5)]
        self.launches_per_step = 7 if world == 1 else 8

    def _setup_peer_buffers(self, dev):
        """Receive buffer, expert-output buffer, counts table and flags in symmetric (peer-mapped) memory."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        t = self.torch
        d, E, W = self.d, self.E, self.world
        sizes = [self.max_rows * d * 2, self.max_rows * d * 4, W * E * 4, 4096]
        self._symm, ptrs = [], []
        for nbytes in sizes:
            buf = symm_mem.empty(nbytes, dtype=t.uint8, device=dev)
            hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
            buf.zero_()
            self._symm.append((buf, hdl))
            ptrs.append(t.tensor([int(p) for p in hdl.buffer_ptrs], dtype=t.int64, device=dev))
        self.peer_recv_x, self.peer_ffn_out, self.peer_counts, self.peer_flags = ptrs
        self.recv_x = self._symm[0][0].view(t.bfloat16)
        self.ffn_out = self._symm[1][0].view(t.float32)
        t.cuda.synchronize()
        dist.barrier()

    # ---- host-side loading -------------------------------------------------------------
    def load(self, x_bits, wg_bits, w1_bits, w2_bits):
        """x: this rank's tokens; w1/w2: this rank's experts; all as uint16 bf16 bits."""
        t = self.torch
        for dst, src in ((self.x, x_bits), (self.wg, wg_bits), (self.w1, w1_bits), (self.w2, w2_bits)):
            dst.view(t.int16).copy_(t.from_numpy(np.ascontiguousarray(src).view(np.int16)))

    # ---- one step ------------------------------------------------------------------------
    def ffn_rows(self):
        """Rows the expert FFN of this rank processed in the last pass (device read; synchronises)."""
        off = self.group_offsets if self.world > 1 else self.offsets
        return int(off[-1].item())

    def forward(self, stream=None):
        """Enqueues one layer pass on `stream` (default: the layer's stream) and returns the output tensor."""
        s = stream or self.stream
        self.k_gate.launch(s)
        self.k_top2.launch(s)
        self.k_weights.launch(s)
        if self.world == 1:
            self.k_ffn.launch(s)
            self.k_combine.launch(s)
        elif self.exchange == "peer":
            self.k_phase[0].launch(s)   # counts exchange + rows to their experts' ranks
            self.k_phase[1].launch(s)   # wait for every source's rows
            self.k_ffn.launch(s)
            self.k_phase[2].launch(s)   # expert outputs ready
            self.k_phase[3].launch(s)   # pull and combine
            self.k_phase[4].launch(s)   # advance the pass number
        else:
            self._exchange_forward()
            self.k_combine.launch(s)
        return self.out

    # ---- CUDA graph of one pass ---------------------------------------------------------
    def capture(self):
        """Captures one pass into a CUDA graph (every exchange mode except "nccl", whose split sizes
        need the host).  Call after at least one eager pass.  Returns False when not capturable."""
        if self.exchange == "nccl":
            return False
        t = self.torch
        self._side = t.cuda.Stream()
        self._side_stream = self.ctx.wrap_stream(self._side.cuda_stream)
        self._graph = t.cuda.CUDAGraph()
        t.cuda.synchronize()
        with t.cuda.graph(self._graph, stream=self._side):
            self.forward(self._side_stream)
        return True

    def replay(self):
        self._graph.replay()
        return self.out

    def _exchange_forward(self):
        t, dist = self.torch, self.torch.distributed
        s, d = self.stream, self.d
        self.k_compact.launch(s)
        dist.all_gather_into_tensor(self.counts_all, self.requested)
        self.host_counts.copy_(self.counts_all, non_blocking=True)
        t.cuda.current_stream().synchronize()
        counts = self.host_counts.numpy().reshape(self.world, self.E)
        send_rows, recv_rows, group_offsets = split_plan(counts, self.rank, self.world)
        self.host_group_offsets.numpy()[:] = group_offsets.view(np.int32)
        self.group_offsets.copy_(self.host_group_offsets, non_blocking=True)
        n_send, n_recv = sum(send_rows), sum(recv_rows)
        dist.all_to_all_single(self.recv_x[: n_recv * d], self.compact_x[: n_send * d],
                               [r * d for r in recv_rows], [r * d for r in send_rows])
        self.k_ffn.launch(s)
        dist.all_to_all_single(self.compact_out[: n_send * d], self.ffn_out[: n_recv * d],
                               [r * d for r in send_rows], [r * d for r in recv_rows])
