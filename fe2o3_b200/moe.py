"""MoE top-2 layer: gate -> top-2 routing -> route weights -> expert FFN -> combine.

Single GPU: the host schedule of examples/moe_expert_v1/src/pipeline.rs:166-270
(compact accepted routes by expert, run the experts, inverse-permute, combine in
rank order) with every stage a launch through the C ABI.

Several GPUs (one process per GPU, `torch.distributed`): tokens are split
across ranks and experts are block-partitioned.  Each rank routes its own
tokens; rows bound for experts on other ranks are stored straight into the
owners' receive buffers over NVLink by the dispatch kernel, the owning rank
runs the grouped FFN, whose second GEMM stores every output row into the home
rank's return buffer from its epilogue, and the home rank combines the two rows
of each token in rank order from local memory (`exchange="peer"`, kernels of
csrc/moe_ep.cu and csrc/gemm_tc.cu).  `exchange="nccl"` does the two transfers
with NCCL all-to-alls instead and needs the host for its split sizes.  torch is
used for device memory and process-group plumbing only; every arithmetic stage
is a kernel of libfe2o3_b200.so.
"""
import os

import numpy as np

from . import SCHEDULE_AUTO, Fe2o3Error, PeerRegion, prepare  # noqa: F401

DROP = 0xFFFFFFFF


def split_plan(counts, rank, world):
    """Pure host logic of the NCCL exchange, from the gathered per-(source rank,
    expert) ADMITTED route counts `counts[world][experts]` (the rows that exist
    in the senders' compact buffers: requests beyond an expert's capacity are
    dropped before the exchange).

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


def pair_plan(counts, rank, world):
    """Pure host statement of the peer exchange's row layout, from the same
    admitted counts: on its owner `o`, the rows of local expert `le` are one
    segment made of one run per source, the owner's own rows first, then the
    sources o+1, o+2, ... (mod world): run k (source (o + k) % world) starts at
    pair_offsets[le * world + k].  `bases[e]` is the first row of THIS rank's rows
    for expert e on e's owner.  A rank's own rows for its first local expert start
    at row 0 whatever the other ranks send, which is why the dispatch kernel can
    store them before the counts have been exchanged.  The dispatch kernel computes
    both tables on the device; tests compare against this."""
    counts = np.asarray(counts, np.int64)
    experts = counts.shape[1]
    per = experts // world
    order = [(rank + k) % world for k in range(world)]
    mine = counts[order][:, rank * per:(rank + 1) * per]     # [run k][local expert]
    pair_offsets = np.zeros(experts + 1, np.uint32)
    pair_offsets[1:] = np.cumsum(mine.T.reshape(-1))          # le-major, run-minor
    bases = np.zeros(experts, np.int64)
    for e in range(experts):
        d, le = divmod(e, per)
        k_me = (rank - d) % world
        bases[e] = counts[:, d * per:d * per + le].sum() + sum(counts[(d + k) % world, e] for k in range(k_me))
    return pair_offsets, bases


class MoeTop2Layer:
    def __init__(self, ctx, stream, tokens, d_model, d_ff, experts, rank=0, world=1, capacity=None, exchange="auto",
                 spin_limit=0, peer_ptrs=None, io_sets=1):
        """`io_sets`: how many (input, output) buffer pairs the layer owns (`x_bufs[i]`, `out_bufs[i]`); a pass
        names the pair it reads and writes (`forward(io=i)`), so a host can fill the next pass's input and
        drain the previous pass's output on copy streams while this one computes.
        `peer_ptrs` (optional, peer exchange only): {"recv_x" | "recv_meta" | "ret" | "counts" | "flags":
        [address of rank p's buffer for p in range(world)]} when the caller has mapped the buffers itself
        (sizes: `region_sizes`); by default the layer allocates and maps them."""
        import torch
        self.torch = torch
        # a single rank runs the reference's host schedule unless the peer path is asked for by name
        self.exchange = "none" if (world == 1 and exchange != "peer") else exchange
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
        # tokens in and combined output out are library-owned buffers (the host copies of an end-to-end step
        # go through fe2o3_buf_copy_*_async); the torch tensors are views of the same memory
        from . import DeviceBuffer
        self.x_bufs = [DeviceBuffer.zeroed(stream, T * d, np.uint16) for _ in range(io_sets)]
        self.out_bufs = [DeviceBuffer.zeroed(stream, T * d, np.float32) for _ in range(io_sets)]
        self.xs = [torch.as_tensor(b, device=dev).view(torch.bfloat16) for b in self.x_bufs]
        self.outs = [torch.as_tensor(b, device=dev) for b in self.out_bufs]
        self.x_buf, self.out_buf, self.x, self.out = self.x_bufs[0], self.out_bufs[0], self.xs[0], self.outs[0]
        self.wg = z(d * E, torch.bfloat16)
        self.w1 = z(self.per * d * f, torch.bfloat16)   # this rank's experts only
        self.w2 = z(self.per * f * d, torch.bfloat16)
        self.logits = z(T * E, torch.float32)
        self.top2, self.slots, self.perm, self.inverse = (z(R, torch.int32) for _ in range(4))
        self.requested, self.admitted = z(E, torch.int32), z(E, torch.int32)
        self.offsets = z(E + 1, torch.int32)
        self.weights = z(R, torch.float32)
        # rows this rank may have to process: every admitted route of every rank in the worst case
        self.max_rows = min(R, E * self.capacity) * world
        if self.exchange in ("auto", "peer"):
            try:
                self._setup_peer_buffers(dev, peer_ptrs)
                self.exchange = "peer"
            except Exception as err:  # no peer mapping available: use the NCCL all-to-all path
                if self.exchange == "peer":
                    raise
                self.exchange, self.exchange_fallback_reason = "nccl", f"{type(err).__name__}: {err}"
        P = lambda op, **kw: prepare(ctx, op, **kw)
        # kernels that read the tokens or write the output exist once per buffer pair
        self.k_gates = [P("moe_gate_v1", x=x, wg=self.wg, logits=self.logits, tokens=T, d_model=d, experts=E)
                        for x in self.xs]
        self.k_gate = self.k_gates[0]
        self.k_top2 = P("moe_top2_v1", logits=self.logits, top2_experts=self.top2, requested_counts=self.requested,
                        admitted_counts=self.admitted, expert_offsets=self.offsets, route_slots=self.slots,
                        permutation=self.perm, inverse=self.inverse, tokens=T, experts=E, capacity=self.capacity)
        self.k_weights = P("moe_route_weights_v1", logits=self.logits, top2_experts=self.top2,
                           route_weights=self.weights, tokens=T, experts=E)
        if self.exchange == "peer":
            self.rows = self.max_rows
            self.hidden = z(self.max_rows * f, torch.bfloat16)
            self.pair_offsets = z(E + 1, torch.int32)
            self.epoch_counter = z(1, torch.int32)  # pass number, advanced on the device: passes replay from a graph
            self.progress = z(2 * (self.max_rows // 128 + self.per + 1), torch.int32)   # row-tile hand-over between the FFN GEMMs
            me = rank
            common = dict(pair_offsets=self.pair_offsets, peer_ret=self.peer_ret, peer_flags=self.peer_flags,
                          epoch_counter=self.epoch_counter, tokens=T, d_model=d, experts=E, world=world, rank=rank,
                          epoch=0, max_rows=self.max_rows, spin_limit=spin_limit)
            self.k_phases = [[P("moe_ep_exchange_v1", x=x, top2_experts=self.top2, permutation=self.perm,
                                inverse=self.inverse, expert_offsets=self.offsets, admitted_counts=self.admitted,
                                route_weights=self.weights, combined_output=out, peer_recv_x=self.peer_recv_x,
                                peer_recv_meta=self.peer_recv_meta, peer_counts=self.peer_counts, phase=ph,
                                logits=self.logits if ph == 0 else None, **common)   # dispatch also writes the route weights
                              for ph in range(2)] for x, out in zip(self.xs, self.outs)]
            self.k_phase = self.k_phases[0]
            self.k_ffn = P("moe_ep_ffn_v1", recv_x=(self._ptrs["recv_x"][me], self.max_rows * d), w1=self.w1, w2=self.w2,
                           hidden=self.hidden, recv_meta=(self._ptrs["recv_meta"][me], 2 * self.max_rows),
                           flags=(self._ptrs["flags"][me], 5 * world + 6), progress=self.progress, d_ff=f, **common)
            return
        self.compact_x = z(R * d, torch.bfloat16)            # local routes, expert-major
        self.compact_out = z(R * d, torch.float32)           # FFN rows back in local slot order
        if world > 1:   # NCCL all-to-all path
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
        # one GPU: expert FFN and combine as one operation when the row length allows it (the first GEMM gathers
        # its rows, the second adds the weighted rows into the output); FE2O3_MOE_FUSED_COMBINE=0 keeps the
        # reference's separate launches
        self.fused_combine = world == 1 and d % 64 == 0 and os.environ.get("FE2O3_MOE_FUSED_COMBINE") != "0"
        if self.fused_combine:
            self.k_ffns = [P("moe_expert_ffn_combine_v1", x=x, w1=self.w1, w2=self.w2, permutation=self.perm,
                             expert_offsets=self.offsets, route_weights=self.weights, hidden=self.hidden,
                             combined_output=out, tokens=T, d_model=d, d_ff=f, experts=E)
                           for x, out in zip(self.xs, self.outs)]
            self.k_ffn = self.k_ffns[0]
        elif world == 1:
            self.k_ffns = [P("moe_expert_ffn_v1", x=x, w1=self.w1, w2=self.w2, permutation=self.perm,
                             expert_offsets=self.offsets, compact_x=self.compact_x, hidden=self.hidden,
                             compact_output=self.compact_out, tokens=T, d_model=d, d_ff=f, experts=E) for x in self.xs]
            self.k_ffn = self.k_ffns[0]
        else:
            self.k_compacts = [P("moe_compact_v1", x=x, permutation=self.perm, compact_x=self.compact_x,
                                 tokens=T, d_model=d) for x in self.xs]
            self.k_ffn = P("moe_grouped_ffn_v1", compact_x=ffn_in, w1=self.w1, w2=self.w2, group_offsets=ffn_off,
                           hidden=self.hidden, compact_output=ffn_res, d_model=d, d_ff=f, groups=E,
                           experts_cycle=self.per)
        self.k_combines = [P("moe_expert_combine_v1", compact_output=self.compact_out, inverse=self.inverse,
                             route_weights=self.weights, combined_output=out, tokens=T, width=d) for out in self.outs]
        self.k_combine = self.k_combines[0]

    # ---- peer-visible buffers ---------------------------------------------------------------
    @staticmethod
    def region_sizes(tokens, d_model, experts, world, capacity=None):
        """Bytes of each peer-visible buffer of one rank (tokens = the whole batch)."""
        R = 2 * (tokens // world)
        max_rows = min(R, experts * (R if capacity is None else capacity)) * world
        return {"recv_x": max_rows * d_model * 2, "recv_meta": max_rows * 8, "ret": R * d_model * 4,
                "counts": world * experts * 4, "flags": 4096}

    def _setup_peer_buffers(self, dev, peer_ptrs=None):
        """Receive buffer, row records, return buffer, counts table and flags, mapped by every rank.

        The regions are allocated and exported by the library (fe2o3_peer_region_*, CUDA IPC) and the
        handles travel over the process group; when that is not possible on this system, torch's
        symmetric memory provides the same mapping."""
        t = self.torch
        sizes = self.region_sizes(self.T * self.world, self.d, self.E, self.world, self.capacity)
        self.peer_mapping = None
        if peer_ptrs is not None:
            self._ptrs = {k: [int(p) for p in peer_ptrs[k]] for k in sizes}
            self.peer_mapping = "caller"
        elif self.world == 1:
            self._local = {k: t.zeros(n, dtype=t.uint8, device=dev) for k, n in sizes.items()}
            self._ptrs = {k: [v.data_ptr()] for k, v in self._local.items()}
            self.peer_mapping = "local"
        else:
            import torch.distributed as dist

            def all_ok(ok):   # every rank must take the same branch: agree on the outcome of each step
                flag = t.tensor([1 if ok else 0], dtype=t.int32, device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                return int(flag.item()) == 1
            reason = ""
            try:
                mine = self._create_regions_ipc(sizes)
            except Fe2o3Error as err:
                mine, reason = None, str(err)
            mapped = False
            if all_ok(mine is not None):
                try:
                    self._ptrs = self._import_regions_ipc(dev, sizes, mine)
                    mapped = True
                except Fe2o3Error as err:
                    reason = str(err)
                mapped = all_ok(mapped)
            if mapped:
                self.peer_mapping = "ipc"
            else:
                self.ipc_fallback_reason = reason or "another rank could not map the regions"
                self._close_regions()
                self._ptrs = self._map_regions_symm(dev, sizes)
                self.peer_mapping = "symmetric_memory"
            t.cuda.synchronize()
            dist.barrier()
        table = lambda k: t.tensor(self._ptrs[k], dtype=t.int64, device=dev)
        self.peer_recv_x, self.peer_recv_meta, self.peer_ret = table("recv_x"), table("recv_meta"), table("ret")
        self.peer_counts, self.peer_flags = table("counts"), table("flags")

    def _create_regions_ipc(self, sizes):
        self._regions = {k: PeerRegion.create(self.ctx, n) for k, n in sizes.items()}
        self._imported = []
        return b"".join(self._regions[k].export() for k in sizes)

    def _import_regions_ipc(self, dev, sizes, mine):
        import torch.distributed as dist
        t, W, me = self.torch, self.world, self.rank
        names = list(sizes)
        local = t.tensor(list(mine), dtype=t.uint8, device=dev)
        everyone = t.empty(W * len(mine), dtype=t.uint8, device=dev)
        dist.all_gather_into_tensor(everyone, local)
        blob = bytes(everyone.cpu().numpy())
        ptrs = {k: [0] * W for k in names}
        hb = PeerRegion.HANDLE_BYTES
        for p in range(W):
            for i, k in enumerate(names):
                if p == me:
                    ptrs[k][p] = self._regions[k].ptr
                else:
                    off = p * len(mine) + i * hb
                    region = PeerRegion.open(self.ctx, blob[off:off + hb])
                    self._imported.append(region)
                    ptrs[k][p] = region.ptr
        return ptrs

    def _map_regions_symm(self, dev, sizes):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        t = self.torch
        self._symm, ptrs = [], {}
        for k, nbytes in sizes.items():
            buf = symm_mem.empty(nbytes, dtype=t.uint8, device=dev)
            hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
            buf.zero_()
            self._symm.append((buf, hdl))
            ptrs[k] = [int(p) for p in hdl.buffer_ptrs]
        return ptrs

    def _close_regions(self):
        for r in getattr(self, "_imported", []):
            try:
                r.close()
            except Fe2o3Error:
                pass
        for r in getattr(self, "_regions", {}).values():
            try:
                r.close()
            except Fe2o3Error:
                pass
        self._imported, self._regions = [], {}

    def close(self):
        """Unmaps the other ranks' regions and frees this rank's (call on every rank, after a barrier)."""
        self.torch.cuda.synchronize()
        self._close_regions()

    # ---- host-side loading -------------------------------------------------------------
    def load(self, x_bits, wg_bits, w1_bits, w2_bits):
        """x: this rank's tokens; w1/w2: this rank's experts; all as uint16 bf16 bits."""
        t = self.torch
        for dst, src in ((self.x, x_bits), (self.wg, wg_bits), (self.w1, w1_bits), (self.w2, w2_bits)):
            dst.view(t.int16).copy_(t.from_numpy(np.ascontiguousarray(src).view(np.int16)))

    # ---- one step ------------------------------------------------------------------------
    def ffn_rows(self):
        """Rows the expert FFN of this rank processed in the last pass (device read; synchronises)."""
        if self.exchange == "peer":
            off = self.pair_offsets
        else:
            off = self.group_offsets if self.world > 1 else self.offsets
        return int(off[-1].item())

    def forward(self, stream=None, ffn_marks=None, io=0):
        """Enqueues one layer pass on `stream` (default: the layer's stream) over buffer pair `io` and returns
        the output tensor.  `ffn_marks`: optional (begin, end) events recorded around the expert FFN (one GPU, or
        the peer exchange)."""
        s = stream or self.stream
        self.k_gates[io].launch(s)
        self.k_top2.launch(s)
        if self.exchange != "peer":
            self.k_weights.launch(s)
        if self.exchange == "peer":
            self.k_phases[io][0].launch(s)   # counts exchange + route weights + rows to their experts' ranks
            if ffn_marks:
                ffn_marks[0].record(s)
            self.k_ffn.launch(s)        # waits per source inside; returns rows to their home ranks
            if ffn_marks:
                ffn_marks[1].record(s)
            self.k_phases[io][1].launch(s)   # combine from the local return buffer, advance the pass number
        elif self.world == 1:
            if ffn_marks:
                ffn_marks[0].record(s)
            self.k_ffns[io].launch(s)
            if ffn_marks:
                ffn_marks[1].record(s)
            if not self.fused_combine:
                self.k_combines[io].launch(s)
        else:
            self._exchange_forward(io)
            self.k_combines[io].launch(s)
        return self.outs[io]

    # ---- CUDA graph of one pass ---------------------------------------------------------
    def capture(self):
        """Captures one pass into a CUDA graph (every exchange mode except "nccl", whose split sizes
        need the host).  Call after at least one eager pass.  Returns False when not capturable."""
        if self.exchange == "nccl":
            return False
        t = self.torch
        self._side = t.cuda.Stream()
        self._side_stream = self.ctx.wrap_stream(self._side.cuda_stream)
        self._graphs = []
        for io in range(len(self.xs)):   # one graph per buffer pair
            g = t.cuda.CUDAGraph()
            t.cuda.synchronize()
            with t.cuda.graph(g, stream=self._side):
                self.forward(self._side_stream, io=io)
            self._graphs.append(g)
        return True

    def replay(self, io=0):
        self._graphs[io].replay()
        return self.outs[io]

    def _exchange_forward(self, io=0):
        t, dist = self.torch, self.torch.distributed
        s, d = self.stream, self.d
        self.k_compacts[io].launch(s)
        # the compact buffers hold ADMITTED rows only (expert_offsets is the scan of the admitted counts)
        dist.all_gather_into_tensor(self.counts_all, self.admitted)
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
