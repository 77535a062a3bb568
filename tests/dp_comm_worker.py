"""Worker (torchrun, 2+ GPUs): the peer-memory reduce-scatter / all-gather of the distributed optimizer against
torch.distributed — raw buffers first, then two training steps of a tiny model with the kernels on and off."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mcore_bridge_b200.ops import _lib
from mcore_bridge_b200.parallel import dp_comm
from mcore_bridge_b200.parallel import state as ps

ps.init_distributed()
world, rank = dist.get_world_size(), dist.get_rank()
ps.initialize_model_parallel()
dev = torch.device('cuda', torch.cuda.current_device())
ok = True


def agree(good: bool) -> bool:
    t = torch.tensor([0 if good else 1], device=dev)
    dist.all_reduce(t)
    return t.item() == 0


def timed(fn, iters=5):
    fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


assert dp_comm.usable('dp', dev), 'the peer-memory path must be available on a multi-GPU box'
unit = 128 * world
numel = unit * 40000 + unit * 3            # two buckets of different size
cut = unit * 40000
ws, grad = dp_comm.allocate('dp', numel, torch.float32)
g = torch.Generator(device=dev).manual_seed(7 + rank)
src = torch.randn(numel, device=dev, generator=g)
ref = src.clone()
dist.all_reduce(ref)
for rep in range(3):                        # repeated calls reuse the flags with a new epoch
    grad.copy_(src)
    torch.cuda.synchronize()
    dist.barrier()
    for s, e in ((0, cut), (cut, numel)):
        dp_comm.reduce_scatter_(ws, grad, s, e)
        n = (e - s) // world
        mine = slice(s + rank * n, s + (rank + 1) * n)
        good = torch.allclose(grad[mine], ref[mine], rtol=1e-6, atol=1e-6)
        if world == 2:
            good = good and torch.equal(grad[mine], ref[mine])
        # everything outside this rank's slice is untouched
        other = torch.ones(numel, dtype=torch.bool, device=dev)
        other[mine] = False
        if (s, e) == (0, cut):
            good = good and torch.equal(grad[other], src[other])
        ok &= agree(good)
torch.cuda.synchronize()
_lib.check_status()
if rank == 0:
    print('reduce-scatter', 'OK' if ok else 'FAIL', flush=True)

ws2, par = dp_comm.allocate('dp', numel, torch.bfloat16)
full = torch.randn(numel, device=dev, generator=torch.Generator(device=dev).manual_seed(3)).to(torch.bfloat16)
for rep in range(2):
    par.zero_()
    for s, e in ((0, cut), (cut, numel)):
        n = (e - s) // world
        par[s + rank * n:s + (rank + 1) * n] = full[s + rank * n:s + (rank + 1) * n]
    torch.cuda.synchronize()
    dist.barrier()
    for s, e in ((0, cut), (cut, numel)):
        dp_comm.all_gather_(ws2, par, s, e)
    ok &= agree(torch.equal(par, full))
torch.cuda.synchronize()
_lib.check_status()
if rank == 0:
    print('all-gather', 'OK' if ok else 'FAIL', flush=True)

# timing of one 256 MiB gradient bucket and the matching bf16 parameter bucket against the library collectives
big = 64 * 1024 * 1024 // unit * unit
wsb, gb = dp_comm.allocate('dp', big, torch.float32)
wsp, pb = dp_comm.allocate('dp', big, torch.bfloat16)
plain_g, plain_p = torch.randn(big, device=dev), torch.zeros(big, dtype=torch.bfloat16, device=dev)
n = big // world
t_rs = timed(lambda: dp_comm.reduce_scatter_(wsb, gb, 0, big))
t_rs_lib = timed(lambda: dist.reduce_scatter_tensor(plain_g[rank * n:(rank + 1) * n], plain_g))
t_ag = timed(lambda: dp_comm.all_gather_(wsp, pb, 0, big))
t_ag_lib = timed(lambda: dist.all_gather_into_tensor(plain_p, plain_p[rank * n:(rank + 1) * n]))
_lib.check_status()
if rank == 0:
    link = (world - 1) / world
    print(f'TIMING world={world} reduce_scatter fp32 {big * 4 >> 20} MiB: peer kernel {t_rs:.3f} ms '
          f'({big * 4 * link / t_rs / 1e6:.0f} GB/s in), library {t_rs_lib:.3f} ms; all_gather bf16 {big * 2 >> 20} MiB: '
          f'peer kernel {t_ag:.3f} ms ({big * 2 * link / t_ag / 1e6:.0f} GB/s in), library {t_ag_lib:.3f} ms', flush=True)

# two optimizer steps of a tiny model, data parallel over all ranks: kernels on vs off
from mcore_bridge_b200.train.data import SyntheticPackedDataset
from mcore_bridge_b200.train.presets import model_config
from mcore_bridge_b200.train.trainer import TrainConfig, Trainer

def run_steps(flag: str, overlap: bool = True):
    """Two optimizer steps; returns the losses, the flat parameters after each step and whether the peer-memory
    buffers were in use."""
    os.environ['MCB200_FUSED_DP'] = flag
    torch.manual_seed(0)
    cfg = model_config('qwen3_tiny', bf16=True)
    trainer = Trainer(cfg, TrainConfig(lr=1e-3, overlap_grad_reduce=overlap))
    used = any(buf.fused for m in trainer.ddp for buf in m.buffers.values())
    ds = SyntheticPackedDataset(cfg.padded_vocab_size, 1024, seg_lo=128, seg_hi=512, seed=11 + rank)
    losses, flats = [], []
    for _ in range(2):
        losses.append(trainer.train_step([ds.next_microbatch() for _ in range(2)]))
        flats.append(torch.cat([p.detach().float().reshape(-1) for m in trainer.models for p in m.parameters()]))
    torch.cuda.synchronize()
    _lib.check_status()
    names = [(n, p.numel()) for m in trainer.models for n, p in m.named_parameters()]
    return losses, flats, used, names


# The library path twice gives the run-to-run noise of the step itself (atomics in a few gradient kernels plus Adam's
# first steps, which turn a rounding-level difference of a near-zero gradient into a full +-lr update); the
# peer-memory path has to stay within it.
fused, lib_a, lib_b = run_steps('1'), run_steps('0'), run_steps('0')
def dist_of(x, y):
    return [(p - q).abs().max().item() for p, q in zip(x[1], y[1])], [abs(p - q) for p, q in zip(x[0], y[0])]


noise_p, noise_l = dist_of(lib_a, lib_b)
diff_p, diff_l = dist_of(fused, lib_a)
frac = [((p - q).abs() > 1e-6).float().mean().item() for p, q in zip(fused[1], lib_a[1])]
frac_noise = [((p - q).abs() > 1e-6).float().mean().item() for p, q in zip(lib_a[1], lib_b[1])]
good = fused[2] and not lib_a[2]
good = good and diff_l[0] < 1e-6 and diff_l[1] < 2e-4          # the first loss only depends on the forward pass
good = good and all(f <= 2 * n + 1e-3 for f, n in zip(frac, frac_noise))
good = good and all(d <= 2 * n + 1e-6 for d, n in zip(diff_p, noise_p))
ok &= agree(good)
if rank == 0:
    print(f'training steps: losses fused {fused[0]} library {lib_a[0]} / {lib_b[0]}; max |dparam| fused-vs-library '
          f'{diff_p} (fraction differing {frac}), library-vs-library {noise_p} (fraction {frac_noise})',
          'OK' if good else 'FAIL', flush=True)
    print('ALL OK' if ok else 'SOME FAILED', flush=True)
