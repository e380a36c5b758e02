"""Check of the peer-memory kernels against NCCL on 2, 4 or 8 ranks (run under torchrun).

Also exercises failure detection the safe way: a wait on a flag that nothing
sets, with a short polling budget, must return with status 5 (peer timeout) and
leave the context usable.
"""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from systems_for_llms_b200.ops.gemm import check_status, status_word  # noqa: E402
from systems_for_llms_b200.parallel.comm import PeerComm, SymmetricBuffer  # noqa: E402

rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
out = {}
comm = PeerComm(dev, ctas=16)
n = 4_000_000
buf = SymmetricBuffer(n * 4, dev)
g = buf.view(torch.float32, n)
torch.manual_seed(rank)
src = torch.randn(n, device=dev)
g.copy_(src)
ref = src.clone()
dist.all_reduce(ref)
ref /= world
dist.barrier()
torch.cuda.synchronize()
comm.allreduce(buf, 0, n, 1.0 / world, 0)
torch.cuda.synchronize()
check_status()
out["allreduce_maxerr"] = (g - ref).abs().max().item()
sums = [None] * world
dist.all_gather_object(sums, g.double().sum().item())
out["replicas_equal"] = len(set(sums)) == 1
stats = comm.norm_finalize(buf, torch.tensor([0], dtype=torch.int32, device=dev), 1.0)
out["norm"], out["norm_ref"] = stats[0].item(), torch.linalg.vector_norm(ref).item()

g.copy_(src)
pbuf, sbuf = SymmetricBuffer(n * 4, dev), SymmetricBuffer(n * 2, dev)
p, shadow = pbuf.view(torch.float32, n), sbuf.view(torch.bfloat16, n)
torch.manual_seed(123)
p0 = torch.randn(n, device=dev)
p.copy_(p0)
per = (n // 4 + world - 1) // world * 4
gs, m, v = (torch.zeros(per, device=dev) for _ in range(3))
dist.barrier()
torch.cuda.synchronize()
comm.reduce_scatter(buf, 0, n, 1.0 / world, gs, 1)
stats = comm.norm_finalize(buf, torch.tensor([1], dtype=torch.int32, device=dev), 0.5)
comm.adamw_allgather(pbuf, sbuf, 0, n, gs, m, v, step=1, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                     weight_decay=0.1, coef=stats[1:2], ok=stats[2:3], slot=2)
torch.cuda.synchronize()
check_status()
pr = torch.nn.Parameter(p0.clone())
pr.grad = ref.clone()
torch.nn.utils.clip_grad_norm_([pr], 0.5)
torch.optim.AdamW([pr], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1).step()
out["zero_param_maxerr"] = (p - pr.detach()).abs().max().item()
out["zero_shadow_ok"] = bool(torch.equal(shadow, p.bfloat16()))

mb = 1 << 20
ab = SymmetricBuffer(world * mb, dev)
a = ab.view(torch.uint8, world * mb)
a.zero_()
a[rank * mb:(rank + 1) * mb] = rank + 1
dist.barrier()
torch.cuda.synchronize()
comm.allgather_bytes(ab, 0, mb, 3)
torch.cuda.synchronize()
check_status()
out["allgather_ok"] = all(bool((a[r * mb:(r + 1) * mb] == r + 1).all()) for r in range(world))

rows, cols = 1024, 512
pb, ob = SymmetricBuffer(rows * cols * 2, dev), SymmetricBuffer(rows * cols * 4, dev)
part = pb.view(torch.bfloat16, rows * cols).view(rows, cols)
torch.manual_seed(100 + rank)
part.copy_(torch.randn(rows, cols, device=dev).bfloat16())
torch.manual_seed(7)
resid = torch.randn(rows, cols, device=dev)
total = part.float().clone()
dist.all_reduce(total)
dist.barrier()
torch.cuda.synchronize()
comm.reduce_rows_resid(pb, ob, 0, 0, resid, rows, cols, 4)
torch.cuda.synchronize()
check_status()
got = ob.view(torch.float32, rows * cols).view(rows, cols)
out["tp_reduce_maxerr"] = (got - (resid + total.bfloat16().float())).abs().max().item()

# GEMM fused with its all-reduce: must equal the two-kernel path bit for bit
# (same bf16 partials, same rank-order sum), for both operand layouts, with a
# ragged last row tile, several launches in a row (staging and flag reuse).
from systems_for_llms_b200.ops import gemm as G  # noqa: E402
from systems_for_llms_b200.parallel.tensor_parallel import TensorParallelComm  # noqa: E402

tp = TensorParallelComm(dev, None, num_layers=2)
M, N, KL = 1000, 512, 192
fused_equal, fused_err = True, 0.0
for trial in range(3):
    torch.manual_seed(1000 * trial + rank)
    a = torch.randn(M, KL, device=dev).bfloat16()
    w = (torch.randn(N, KL, device=dev) / KL ** 0.5).bfloat16()
    w_t = w.t().contiguous()                    # [KL, N]: the input-gradient layout
    torch.manual_seed(5 + trial)
    resid = torch.randn(M, N, device=dev)
    two_step = tp.reduce_residual(G.linear_fwd(a, w, tp.partial(M, N)), resid, 0).clone()
    two_step_bf16 = tp.reduce_bf16(G.linear_dgrad(a, w_t, tp.partial(M, N))).clone()
    one_step = tp.gemm_reduce_residual(a, w, resid, 1).clone()
    one_step_bf16 = tp.gemm_reduce_bf16(a, w_t).clone()
    torch.cuda.synchronize()
    check_status()
    fused_equal &= bool(torch.equal(one_step, two_step)) and bool(
        torch.equal(one_step_bf16, two_step_bf16))
    exact = a.float() @ w.float().t()
    dist.all_reduce(exact)
    fused_err = max(fused_err, (one_step - resid - exact).abs().max().item(),
                    (one_step_bf16.float() - exact).abs().max().item())
out["tp_fused_equal"], out["tp_fused_maxerr"] = fused_equal, fused_err
replicas = [None] * world
dist.all_gather_object(replicas, (one_step.double().sum().item(), one_step_bf16.double().sum().item()))
out["tp_fused_replicas_equal"] = len(set(replicas)) == 1
dist.barrier()
torch.cuda.synchronize()
tp.close()

# Failure detection without faulting anything: only rank 0 enters a collective on
# a fresh slot with a ~1 ms polling budget; the flag it waits for is never set.
dist.barrier()
torch.cuda.synchronize()
comm.set_spin_limit(1 << 12)
if rank == 0:
    comm.allreduce(buf, 0, 1024, 1.0, 40)
    torch.cuda.synchronize()
    out["timeout_status"] = int(status_word(dev).item())
    status_word(dev).zero_()
else:
    out["timeout_status"] = 5
comm.set_spin_limit(48 << 20)
dist.barrier()
# the context is still usable and the slot works again once everybody joins
if rank != 0:
    comm._epochs[40] += 1      # rank 0 already consumed one epoch of slot 40
buf.view(torch.float32, 1024).fill_(1.0)
dist.barrier()
torch.cuda.synchronize()
comm.allreduce(buf, 0, 1024, 1.0, 40)       # the slot whose wait ran out, not a fresh one
torch.cuda.synchronize()
out["recovered_after_timeout"] = bool((buf.view(torch.float32, 1024) == world).all().item())
check_status()
dist.barrier()
if rank == 0:
    with open(sys.argv[1], "w") as handle:
        json.dump(out, handle)
dist.destroy_process_group()
