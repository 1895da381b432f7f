"""The expert-parallel MoE layer (peer exchange) on ONE GPU.

A single rank can run the whole peer path against its own buffers.  Several
ranks are run here as "virtual ranks" in one process, one after another: every
rank's kernels find the flags they wait for already raised (the host publishes
the counts table that the ranks' dispatch kernels would exchange, and rank r's
rows, outputs and flags are complete before the next stage starts), so no kernel
ever waits for another kernel, while every index computation of the world-size-W
layout (row bases on the owners, (local expert, source) pairs, per-source waits,
the scatter of output rows to their home ranks) runs exactly as it does with W
processes.  Routing is compared bit-for-bit and outputs within BASELINE's
tolerance against the CPU oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SPIN = 2000  # polls before a device-side wait gives up: nothing here should ever have to wait


@pytest.fixture(scope="module")
def gpu():
    import fe2o3_b200 as fe
    ctx = fe.GpuContext(0)
    return fe, ctx, ctx.default_stream()


def _inputs(T, d, f, E):
    from fe2o3_b200 import synth
    x = synth.normal_bf16(4, 1, T * d, 1.0)
    wg = synth.normal_bf16(4, 2, d * E, 0.02)
    w1 = np.concatenate([synth.normal_bf16(4, 100 + e, d * f, 0.02) for e in range(E)])
    w2 = np.concatenate([synth.normal_bf16(4, 200 + e, f * d, 0.02) for e in range(E)])
    return x, wg, w1, w2


def _oracle_rank(orc, x, wg, w1, w2, T, d, f, E, capacity):
    """One rank's tokens through the oracle with that rank's capacity (drops are per rank)."""
    logits = orc.moe_gate_logits(x, wg, T, d, E)
    _, routing = orc.moe_top2_route(logits, T, E, capacity)
    w = orc.moe_route_weights(logits, routing["top2_experts"], T, E)
    compact = orc.moe_expert_ffn(x, w1, w2, routing["top2_experts"], routing["inverse"], T, d, f, E)
    st, want = orc.moe_combine(compact, routing["inverse"], w, T, d)
    assert st == 0
    return routing, want.reshape(T, d)


def _close(out, want):
    limit = 2e-3 * np.abs(want).max() + 2e-2 * np.abs(want)   # BASELINE rel 2e-2 plus a stated absolute term
    return bool((np.abs(out - want) <= limit).all())


@pytest.mark.parametrize("shape,capacity", [((512, 256, 512, 8), None), ((384, 128, 256, 4), 150), ((200, 64, 128, 8), None)])
def test_peer_path_single_rank(gpu, orc, shape, capacity):
    import torch
    fe, ctx, stream = gpu
    from fe2o3_b200.moe import MoeTop2Layer
    T, d, f, E = shape
    x, wg, w1, w2 = _inputs(T, d, f, E)
    layer = MoeTop2Layer(ctx, stream, T, d, f, E, capacity=capacity, exchange="peer", spin_limit=SPIN)
    assert layer.exchange == "peer" and layer.peer_mapping == "local"
    layer.load(x, wg, w1, w2)
    routing, want = _oracle_rank(orc, x, wg, w1, w2, T, d, f, E, layer.capacity)
    for _ in range(3):   # counters re-arm and the pass number advances on the device
        out = layer.forward().cpu().numpy().reshape(T, d)
        assert ctx.take_kernel_status(stream) == 0
        assert (layer.top2.cpu().numpy().view(np.uint32) == routing["top2_experts"]).all()
        assert (layer.inverse.cpu().numpy().view(np.uint32) == routing["inverse"]).all()
        assert _close(out, want), float(np.abs(out - want).max())
    assert int(layer.epoch_counter.item()) == 3
    # the same pass replayed from a CUDA graph
    assert layer.capture()
    layer.out.zero_()
    out = layer.replay().cpu().numpy().reshape(T, d)
    torch.cuda.synchronize()
    assert ctx.take_kernel_status(stream) == 0 and _close(out, want)


@pytest.mark.parametrize("shape,capacity", [((512, 128, 256, 8), None), ((700, 192, 320, 4), 260), ((300, 136, 256, 8), None)])
def test_single_gpu_layer_fused_and_separate_schedules_agree(gpu, orc, monkeypatch, shape, capacity):
    """One GPU: the layer runs gate, routing, route weights and the expert FFN with the combine folded in
    (six launches); with FE2O3_MOE_FUSED_COMBINE=0, or a row length that is not whole 64-column blocks, it
    runs the reference's schedule (compaction or gathered rows, two GEMMs, combine kernel).  Same bits, both
    replayed from CUDA graphs over two input/output buffer pairs, and the oracle's result within tolerance."""
    fe, ctx, stream = gpu
    import torch
    from fe2o3_b200.moe import MoeTop2Layer
    T, d, f, E = shape
    x, wg, w1, w2 = _inputs(T, d, f, E)
    outs = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("FE2O3_MOE_FUSED_COMBINE", mode)
        layer = MoeTop2Layer(ctx, stream, T, d, f, E, capacity=capacity, io_sets=2)
        assert layer.fused_combine == (mode == "1" and d % 64 == 0)
        layer.load(x, wg, w1, w2)
        layer.xs[1].copy_(layer.xs[0])
        first = layer.forward().cpu().numpy().copy()
        assert ctx.take_kernel_status(stream) == 0
        assert layer.capture()
        for io in (0, 1, 0):
            layer.outs[io].fill_(float("nan"))
            got = layer.replay(io=io).cpu().numpy()
            torch.cuda.synchronize()
            assert (got.view(np.uint32) == first.view(np.uint32)).all()
        outs[mode] = first
    assert (outs["0"].view(np.uint32) == outs["1"].view(np.uint32)).all()
    _, want = _oracle_rank(orc, x, wg, w1, w2, T, d, f, E, T * 2 if capacity is None else capacity)
    assert _close(outs["1"].reshape(T, d), want)


class VirtualRanks:
    """W ranks of the peer exchange in one process on one GPU, stepped stage by stage."""

    def __init__(self, fe, ctx, stream, shape, world, capacity=None):
        import torch
        from fe2o3_b200.moe import MoeTop2Layer
        T, d, f, E = shape
        self.torch, self.world, self.shape = torch, world, shape
        sizes = MoeTop2Layer.region_sizes(T, d, E, world, capacity)
        self.bufs = [{k: torch.zeros(n, dtype=torch.uint8, device="cuda") for k, n in sizes.items()} for _ in range(world)]
        ptrs = {k: [self.bufs[r][k].data_ptr() for r in range(world)] for k in sizes}
        self.layers = [MoeTop2Layer(ctx, stream, T, d, f, E, rank=r, world=world, capacity=capacity, exchange="peer",
                                    spin_limit=SPIN, peer_ptrs=ptrs) for r in range(world)]
        self.stream, self.epoch = stream, 0

    def load(self, x, wg, w1, w2):
        T, d, f, E = self.shape
        tl, per = T // self.world, E // self.world
        for r, layer in enumerate(self.layers):
            layer.load(x[r * tl * d:(r + 1) * tl * d], wg, w1[r * per * d * f:(r + 1) * per * d * f],
                       w2[r * per * f * d:(r + 1) * per * f * d])

    def step(self):
        t, s, W = self.torch, self.stream, self.world
        E = self.shape[3]
        self.epoch += 1
        for layer in self.layers:
            layer.k_gate.launch(s)
            layer.k_top2.launch(s)   # the route weights are written by the dispatch kernel
        # what the dispatch kernels' first blocks would exchange: every rank's admitted counts in every
        # rank's table, and the "counts published" flags at this pass's epoch
        counts = t.stack([layer.admitted for layer in self.layers]).reshape(-1)            # [W][E] int32
        for r in range(W):
            self.bufs[r]["counts"].view(t.int32)[: W * E].copy_(counts)
            self.bufs[r]["flags"].view(t.int32)[:W].fill_(self.epoch)
        for layer in self.layers:
            layer.k_phase[0].launch(s)
        for layer in self.layers:
            layer.k_ffn.launch(s)
        for layer in self.layers:
            layer.k_phase[1].launch(s)
        t.cuda.synchronize()
        return counts.cpu().numpy().reshape(W, E)


@pytest.mark.parametrize("world,shape,capacity", [(2, (512, 256, 512, 8), None), (4, (1024, 128, 256, 8), None),
                                                  (8, (2048, 128, 256, 8), None), (2, (512, 128, 256, 4), 100),
                                                  (4, (520, 64, 128, 16), None)])
def test_virtual_ranks_match_oracle(gpu, orc, world, shape, capacity):
    fe, ctx, stream = gpu
    from fe2o3_b200.moe import pair_plan
    T, d, f, E = shape
    x, wg, w1, w2 = _inputs(T, d, f, E)
    vr = VirtualRanks(fe, ctx, stream, shape, world, capacity)
    vr.load(x, wg, w1, w2)
    tl = T // world
    wants = [_oracle_rank(orc, x[r * tl * d:(r + 1) * tl * d], wg, w1, w2, tl, d, f, E, vr.layers[r].capacity)
             for r in range(world)]
    for _ in range(2):
        counts = vr.step()
        assert ctx.take_kernel_status(stream) == 0
        for r, layer in enumerate(vr.layers):
            routing, want = wants[r]
            assert (layer.top2.cpu().numpy().view(np.uint32) == routing["top2_experts"]).all()
            assert (counts[r] == routing["admitted_counts"]).all()
            # the row layout the dispatch kernel derived on the device, against its host statement
            pairs, _ = pair_plan(counts, r, world)
            assert (layer.pair_offsets.cpu().numpy().view(np.uint32) == pairs).all()
            out = layer.out.cpu().numpy().reshape(tl, d)
            assert _close(out, want), (r, float(np.abs(out - want).max()))
            assert int(layer.epoch_counter.item()) == vr.epoch


def test_waits_run_out_and_the_next_pass_works(gpu, orc):
    """Every device-side wait of the exchange gives up after its limit, reports WAIT_EXPIRED through the
    status word and leaves the context usable: the flags waited for here are simply never raised (the pass
    number is set ahead of them), so the kernels return by themselves."""
    fe, ctx, stream = gpu
    from fe2o3_b200.moe import MoeTop2Layer
    T, d, f, E = 256, 128, 256, 8
    x, wg, w1, w2 = _inputs(T, d, f, E)
    layer = MoeTop2Layer(ctx, stream, T, d, f, E, exchange="peer", spin_limit=20000)
    layer.load(x, wg, w1, w2)
    _, want = _oracle_rank(orc, x, wg, w1, w2, T, d, f, E, layer.capacity)
    out = layer.forward().cpu().numpy().reshape(T, d)
    assert ctx.take_kernel_status(stream) == 0 and _close(out, want)
    # pass number 2 is next; pretend it is 7: nobody has raised anything for pass 7
    layer.epoch_counter.fill_(6)
    layer.out.fill_(-1.0)
    for kernel in (layer.k_phase[1], layer.k_ffn):      # combine; FFN (its first GEMM's producer waits for rows)
        with pytest.raises(fe.Fe2o3Error) as err:
            kernel.launch_and_wait(stream, 20000)
        assert err.value.status == -12 and kernel.kernel_status == 4   # KernelStatus, FE2O3_KSTATUS_WAIT_EXPIRED
        layer.epoch_counter.fill_(6)   # the combine advances the pass number even when it gave up
    assert (layer.out.cpu().numpy() == -1.0).all()      # a pass that gave up writes no output
    # back to the true pass number: the counters were re-armed by the kernels that gave up
    layer.epoch_counter.fill_(1)
    out = layer.forward().cpu().numpy().reshape(T, d)
    assert ctx.take_kernel_status(stream) == 0 and _close(out, want)
