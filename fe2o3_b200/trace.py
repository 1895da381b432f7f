"""Device time stamps of the kernels, from a library built with `python fe2o3_b200/build.py --trace`.

    FE2O3_B200_LIB=fe2o3_b200/libfe2o3_b200_trace.so python -m fe2o3_b200.trace attention
    FE2O3_B200_LIB=fe2o3_b200/libfe2o3_b200_trace.so python -m fe2o3_b200.trace moe_peer
    FE2O3_B200_LIB=$PWD/fe2o3_b200/libfe2o3_b200_trace.so python -m torch.distributed.run --nnodes=1 \
        --nproc-per-node N --master-addr 127.0.0.1 --master-port 29713 -m fe2o3_b200.trace moe_ranks

`attention`: SM-clock stamps of CTA 0's softmax warps through the phases of a key block and through its
units, and every CTA's cycles and wall-clock time (csrc/attention_tc.cu, FE2O3_ATTN_TRACE).
`moe_peer`: the timeline of one pass of the expert-parallel MoE kernels on one GPU, the rank being its own
and only peer (csrc/moe_ep.cu and csrc/gemm_tc.cu, FE2O3_EP_TRACE).  `moe_ranks`: the same timeline of every rank of an N-GPU run (one process per
GPU), for one pass replayed from the CUDA graph.
A development aid: the stamps cost a few global stores per block and are compiled out of the normal build.
"""
import ctypes as C
import sys

import numpy as np

EP_STAMPS = ["disp_begin", "counts_here", "rows_sent", "ffn1_begin", "ffn1_first_wait", "ffn1_last_wait", "ffn1_end",
             "ffn2_begin", "ffn2_end", "comb_begin", "outputs_here", "comb_end", "own_rows_done", "ffn1_table"]


def _trace_symbol(lib, name):
    if not hasattr(lib, name):
        raise SystemExit(f"{name} is not in the loaded library: build it with `python fe2o3_b200/build.py --trace` "
                         "and select it with FE2O3_B200_LIB")
    return getattr(lib, name)


def attention(batch=4, heads=16, seq=2048, dim=64):
    import fe2o3_b200 as fe
    from fe2o3_b200 import synth
    from fe2o3_b200._lib import lib
    read = _trace_symbol(lib, "fe2o3_debug_attn_trace")
    read.restype = C.c_int32
    ctx = fe.GpuContext(0)
    stream = ctx.default_stream()
    n = batch * heads * seq * dim
    q, k, v = (fe.DeviceBuffer.from_host(stream, synth.normal_bf16(3, 1 + i, n, 1.0)) for i in range(3))
    out = fe.DeviceBuffer.zeroed(stream, n, np.float32)
    prep = fe.prepare(ctx, "flash_attention_v1", q=q, k=k, v=v, output=out, batch=batch, heads=heads, seq=seq, dim=dim,
                      scale=1.0 / np.sqrt(dim), causal=0, input_dtype=fe.DTYPE_BF16)
    for _ in range(5):
        prep.launch(stream)
    e0, e1 = fe.Event(ctx), fe.Event(ctx)
    e0.record(stream)
    for _ in range(20):
        prep.launch(stream)
    e1.record(stream)
    stream.synchronize()
    ms = e1.elapsed_time_ms_since(e0) / 20
    print(f"{ms * 1e3:.1f} us per launch, {4.0 * batch * heads * seq * seq * dim / ms / 1e9:.0f} TFLOP/s, "
          f"kernel status {ctx.take_kernel_status(stream)}")
    buf = (C.c_ulonglong * 2048)()
    assert read(buf) == 0
    t = np.array(buf[:], dtype=np.int64)
    phases = ["wait", "s_here", "loaded", "max", "exp", "p_stored", "arrived"]
    base = t[:1024][t[:1024] > 0].min()
    for tile in range(2):
        print(f"softmax warps of tile {tile}, first unit, SM cycles since the CTA's first stamp (and per phase)")
        for b in range(2, 7):
            r = t[(tile * 8 + b) * 8:(tile * 8 + b) * 8 + 7] - base
            print(f"  block {b}: " + " ".join(f"{nm}={int(x)}" for nm, x in zip(phases, r)) + f"  {np.diff(r).tolist()}")
    for tile in range(2):
        for unit in range(6):
            r = t[512 + (tile * 8 + unit) * 8:512 + (tile * 8 + unit) * 8 + 4]
            if r[0] > 0:
                print(f"tile {tile} unit {unit}: begin {int(r[0] - base)}, blocks done {int(r[1] - base)}, "
                      f"last P*V done {int(r[2] - base)}, output done {int(r[3] - base) if r[3] > 0 else '-'}")
    ctas = t[1024:].reshape(-1, 4)
    ctas = ctas[ctas[:, 0] > 0]
    cyc, ns = ctas[:, 2] - ctas[:, 0], ctas[:, 3] - ctas[:, 1]
    print(f"{len(ctas)} CTAs: cycles min/median/max {int(cyc.min())}/{int(np.median(cyc))}/{int(cyc.max())}, "
          f"ns {int(ns.min())}/{int(np.median(ns))}/{int(ns.max())}, SM clock GHz "
          f"{(cyc / ns).min():.3f}/{np.median(cyc / ns):.3f}/{(cyc / ns).max():.3f}, "
          f"first start to last end {int(ctas[:, 3].max() - ctas[:, 1].min())} ns")


def moe_peer(tokens=16384, d_model=2048, d_ff=4096, experts=8):
    import torch

    import fe2o3_b200 as fe
    from fe2o3_b200 import synth
    from fe2o3_b200.moe import MoeTop2Layer
    ctx = fe.GpuContext(0)
    s = ctx.default_stream()
    layer = MoeTop2Layer(ctx, s, tokens, d_model, d_ff, experts, exchange="peer")
    layer.load(synth.normal_bf16(4, 1, tokens * d_model, 1.0), synth.normal_bf16(4, 2, d_model * experts, 0.02),
               np.concatenate([synth.normal_bf16(4, 100 + e, d_model * d_ff, 0.02) for e in range(experts)]),
               np.concatenate([synth.normal_bf16(4, 200 + e, d_ff * d_model, 0.02) for e in range(experts)]))
    layer.forward()
    torch.cuda.synchronize()

    def show(tag):
        tr = layer._local["flags"].view(torch.int64)[256:256 + len(EP_STAMPS)].cpu().numpy()
        print(tag, {n: round((int(tr[i]) - int(tr[0])) / 1000.0, 1) for i, n in enumerate(EP_STAMPS) if tr[i] > 0})
    for _ in range(10):
        layer.forward()
    torch.cuda.synchronize()
    show("launched kernel by kernel, us after the dispatch kernel's start:")
    assert layer.capture()
    for _ in range(10):
        layer.replay()
    torch.cuda.synchronize()
    show("replayed from the CUDA graph:")
    assert ctx.take_kernel_status(s) == 0


def moe_ranks(tokens=16384, d_model=2048, d_ff=4096, experts=8):
    import os

    import torch
    import torch.distributed as dist

    import fe2o3_b200 as fe
    from fe2o3_b200 import synth
    from fe2o3_b200.moe import MoeTop2Layer
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = fe.GpuContext(local)
    s = ctx.default_stream()
    t_local, per = tokens // world, experts // world
    layer = MoeTop2Layer(ctx, s, tokens, d_model, d_ff, experts, rank=rank, world=world)
    x = synth.normal_bf16(4, 1, tokens * d_model, 1.0)[rank * t_local * d_model:(rank + 1) * t_local * d_model]
    layer.load(x, synth.normal_bf16(4, 2, d_model * experts, 0.02),
               np.concatenate([synth.normal_bf16(4, 100 + e, d_model * d_ff, 0.02) for e in range(rank * per, (rank + 1) * per)]),
               np.concatenate([synth.normal_bf16(4, 200 + e, d_ff * d_model, 0.02) for e in range(rank * per, (rank + 1) * per)]))
    layer.forward()
    torch.cuda.synchronize()
    dist.barrier()
    assert layer.capture()
    for _ in range(30):
        layer.replay()
    torch.cuda.synchronize()

    class Raw:   # the stamps live behind the flags of this rank's flags region: 64-bit words 256...
        def __init__(self, ptr, n):
            self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i8", "data": (ptr, False), "version": 2}
    tr = torch.as_tensor(Raw(layer._ptrs["flags"][rank] + 2048, len(EP_STAMPS)), device="cuda").cpu().numpy()
    rel = {n: round((int(tr[i]) - int(tr[0])) / 1000.0, 1) for i, n in enumerate(EP_STAMPS) if tr[i] > 0}
    everyone = [None] * world
    dist.all_gather_object(everyone, (rank, rel))
    if rank == 0:
        print("us after each rank's dispatch kernel started:")
        for r, v in everyone:
            print("rank", r, v)
    assert ctx.take_kernel_status(s) == 0
    dist.barrier()
    layer.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else ""
    if what == "attention":
        attention()
    elif what == "moe_peer":
        moe_peer()
    elif what == "moe_ranks":
        moe_ranks()
    else:
        raise SystemExit(__doc__)
