"""Worker for the multi-GPU tensor-parallel test: one process per GPU, launched by test_gpu_tp.py."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

HID, NFF, QOUT, KV, LAYERS, B = 1024, 1536, 1024, 512, 3, 2
WIDE_B = 12


def dims(world):
    """(hidden, n_ff, q_out, kv_out): every rank needs at least one 256-column block of q and of n_ff."""
    return (1024, 1536, 1024, 512) if world <= 4 else (1024, 2304, 2048, 512)


def main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import ferric_b200 as F
    from ferric_b200.stack import DecodeStack, TPPlan, layer_shards
    from test_tp_gloo import full_layer  # same synthetic layers as the CPU test (sizes overridden below)
    import test_tp_gloo as T
    HID, NFF, QOUT, KV = dims(world)
    T.HID, T.NFF, T.QOUT, T.KV = HID, NFF, QOUT, KV

    ctx = F.Context(rank)
    plan = TPPlan.make(world, rank, HID, NFF, QOUT, KV)
    results = {}
    for mode in ("nccl", "fused", "push", "chain"):
        group = None
        if mode != "nccl":
            group = F.TPGroup(ctx, rank, world, B, HID)
            group.connect_with_torch_distributed()
        st = DecodeStack(ctx, plan, n_layers=LAYERS, batch=B,
                         all_reduce=(lambda t: dist.all_reduce(t)) if mode == "nccl" else None, group=group,
                         push=(mode in ("push", "chain")), chain=(mode == "chain"))
        for l in range(LAYERS):
            sh = layer_shards(plan, full_layer(100 + 10 * l))
            st.add_layer(F.QMatrix.from_bytes(ctx, sh["qkv"], 12, plan.q_rows + 2 * plan.kv_rows, HID),
                         F.QMatrix.from_bytes(ctx, sh["o"], 12, HID, plan.q_rows),
                         F.QMatrix.from_bytes(ctx, sh["gate_up"], 12, 2 * plan.ff_rows, HID),
                         F.QMatrix.from_bytes(ctx, sh["down"], 14, HID, plan.ff_rows))
        st.reserve()
        from ferric_b200 import synth
        h0 = torch.from_numpy(synth.activations(B, HID, seed=5)).cuda()
        st.h.copy_(h0)
        eager = st.step().clone()
        st.capture()
        st.h.copy_(h0)
        replay = st.run().clone()
        torch.cuda.synchronize()
        if group is not None:
            group.check()
        results[mode] = (eager.cpu().numpy(), replay.cpu().numpy())
        st.close()
        dist.barrier()
    # the batched decode path (more than 8 rows): NCCL against the library's two-step pushed all-reduce
    wide = {}
    for mode in ("nccl", "wide"):
        group = None
        if mode == "wide":
            group = F.TPGroup(ctx, rank, world, WIDE_B, HID)
            group.connect_with_torch_distributed()
        st = DecodeStack(ctx, plan, n_layers=LAYERS, batch=WIDE_B,
                         all_reduce=(lambda t: dist.all_reduce(t)) if mode == "nccl" else None, group=group)
        for l in range(LAYERS):
            sh = layer_shards(plan, full_layer(100 + 10 * l))
            st.add_layer(F.QMatrix.from_bytes(ctx, sh["qkv"], 12, plan.q_rows + 2 * plan.kv_rows, HID),
                         F.QMatrix.from_bytes(ctx, sh["o"], 12, HID, plan.q_rows),
                         F.QMatrix.from_bytes(ctx, sh["gate_up"], 12, 2 * plan.ff_rows, HID),
                         F.QMatrix.from_bytes(ctx, sh["down"], 14, HID, plan.ff_rows))
        st.reserve()
        h0 = torch.from_numpy(synth.activations(WIDE_B, HID, seed=6)).cuda()
        st.h.copy_(h0)
        eager = st.step().clone()
        st.capture()
        st.h.copy_(h0)
        replay = st.run().clone()
        torch.cuda.synchronize()
        if group is not None:
            group.check()
        wide[mode] = (eager.cpu().numpy(), replay.cpu().numpy())
        st.close()
        dist.barrier()
    if rank == 0:
        np.savez(out + ".wide.npz", nccl=wide["nccl"][0], wide=wide["wide"][0], wide_replay=wide["wide"][1])
    if rank == 0:
        np.savez(out, **{k: v[0] for k, v in results.items()}, **{k + "_replay": v[1] for k, v in results.items()})
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main(int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4])
