"""One rank of the fused K-split exchange test (launched by torchrun from tests/test_ksplit_multigpu.py).

Every rank multiplies its own K slice with the scatter epilogue storing row block g into rank g's staging slot
(peer memory over NVLink, plain TMA stores), the ranks meet at one barrier, and each owner sums its slots and casts.
Checked bit-for-bit against the NCCL reduce-scatter of plain fp32 partials followed by the same cast, and within
1e-2 of the oracle's fp32 product of the whole K range."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.distributed._symmetric_memory as symm

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import gemm_oracle as O          # noqa: E402
from tesserae_b200 import api                # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    m, n, k_total = 1024, 768, 4096
    k = k_total // world
    p = O.make_bf16_problem(m, n, k_total, seed=77, scale=0.5)            # the same full problem on every rank
    k0, klen = api.shard_range(k_total, world, rank, 64)
    assert klen == k
    k1 = k0 + klen
    to_dev = lambda bits: torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).to(dev)
    a, b = to_dev(p["a_bits"][:, k0:k1]), to_dev(p["b_bits"][:, k0:k1])
    rows = m // world
    s = torch.cuda.current_stream().cuda_stream

    plain = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_b0", elem=api.BF16, tile=(128, 256, 64), cta_group=2,
                                        out_elem=api.F32))
    partial = torch.empty((m, n), dtype=torch.float32, device=dev)
    mine = torch.empty((rows, n), dtype=torch.float32, device=dev)
    c_nccl = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
    plain.ksplit_partials(a, b, partial, partial.numel() * 4, m, n, k, 1, stream=s)
    dist.reduce_scatter_tensor(mine, partial, op=dist.ReduceOp.SUM)
    api.reduce_cast_bf16(mine, 1, 0, c_nccl, c_nccl.numel(), stream=s)

    stag = symm.empty((world, rows, n), dtype=torch.float32, device=dev)
    hdl = symm.rendezvous(stag, dist.group.WORLD.group_name)
    stag.fill_(float("nan"))
    hdl.barrier(channel=0)
    scat = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_scatter", elem=api.BF16, tile=(128, 256, 64),
                                       cta_group=2, out_elem=api.F32, scatter=1))
    c_fused = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
    slot = rows * n * 4
    results = []
    for _ in range(2):                                                     # twice: the staging slots are reused
        scat.ksplit_scatter(a, b, [hdl.buffer_ptrs[g] + rank * slot for g in range(world)], rows, m, n, k, stream=s, start_owner=rank)
        hdl.barrier(channel=0)
        api.reduce_cast_bf16(stag, world, rows * n, c_fused, rows * n, stream=s)
        hdl.barrier(channel=0)
        torch.cuda.synchronize()
        want = O.gemm_f32(p["a"], p["b"])[rank * rows:(rank + 1) * rows]
        err = O.rel_error(c_fused.float().cpu().numpy(), want)["max_rel"]
        # 2 ranks: a + b is the same in either order, so the two paths agree to the bit; with more ranks NCCL's
        # summation order is its own and only the tolerance applies
        same = bool(torch.equal(c_nccl.view(torch.int16), c_fused.view(torch.int16)))
        results.append(dict(err=float(err), bit_equal=same, status=plain.status() | scat.status()))
    # The other fusion: every rank ADDS its tiles into the owner's one fp32 buffer (TMA reduce at the destination),
    # so after the barrier the buffer already is the reduce-scattered sum and only the cast remains.  The buffer
    # starts from zeros; it is used twice here, cleared in between.
    acc = symm.empty((rows, n), dtype=torch.float32, device=dev)
    hdl2 = symm.rendezvous(acc, dist.group.WORLD.group_name)
    radd = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_scatter_add", elem=api.BF16, tile=(128, 256, 64),
                                       cta_group=2, out_elem=api.F32, scatter=2))
    c_add = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
    acc.zero_()
    for _ in range(2):
        hdl2.barrier(channel=0)
        radd.ksplit_scatter(a, b, [hdl2.buffer_ptrs[g] for g in range(world)], rows, m, n, k, stream=s, start_owner=rank)
        hdl2.barrier(channel=0)
        api.cast_clear_bf16(acc, c_add, rows * n, stream=s)          # casts and leaves the zeros the next round needs
        hdl2.barrier(channel=0)
        torch.cuda.synchronize()
        err = O.rel_error(c_add.float().cpu().numpy(), want)["max_rel"]
        same = bool(torch.equal(c_nccl.view(torch.int16), c_add.view(torch.int16)))
        results.append(dict(err=float(err), bit_equal=same or world > 2, status=plain.status() | radd.status(), mode="add"))
    out = [None] * world
    dist.all_gather_object(out, results)
    if rank == 0:
        print("RESULT " + json.dumps(dict(world=world, ranks=out)), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
