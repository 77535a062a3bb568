"""torchrun worker: fused AG->GEMM / GEMM->RS vs all_gather / reduce_scatter + fp32 matmul; then a TP=2 training
step with the fused path on against the same step with it off."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mcore_bridge_b200.ops import _lib  # noqa: E402
from mcore_bridge_b200.parallel import fused_comm as fc  # noqa: E402
from mcore_bridge_b200.parallel import mappings as M  # noqa: E402
from mcore_bridge_b200.parallel import state as ps  # noqa: E402


def rel(a, b):
    """Relative Frobenius error; a wrong row or tile also has to show, so the worst row is checked against the
    scale of the reference (a misplaced 128-row block gives a row error of order 1)."""
    a, b = a.float(), b.float()
    whole = ((a - b).norm() / (b.norm() + 1e-9)).item()
    row = ((a - b).norm(dim=-1).max() / (b.norm(dim=-1).mean() + 1e-9)).item()
    return max(whole, row / 4)


def main():
    ps.init_distributed()
    world, rank = dist.get_world_size(), dist.get_rank()
    ps.initialize_model_parallel(tensor_model_parallel_size=world)
    dev = torch.device('cuda', torch.cuda.current_device())
    torch.manual_seed(100 + rank)
    bad = 0
    for it in range(3):   # several epochs exercise the double-buffered workspace
        # the last shape has the row count of a full training micro-batch (16384+ gathered rows, 64+ row blocks per rank)
        shapes = [(128, 512, 256), (256, 1024, 776), (1024, 2048, 768)]
        if it == 0:
            shapes.append((8192 if world == 2 else 4096, 512, 4096))
        for rows, K, N in shapes:
            g = torch.Generator(device=dev).manual_seed(7)
            w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
            x = torch.randn(rows, K, device=dev, dtype=torch.bfloat16)
            y, xg = fc.all_gather_gemm(x, w, None, 'tp')
            xg_ref = M.all_gather_dim0(x, 'tp')
            bad += int(not torch.equal(xg, xg_ref)) + int(rel(y, xg_ref.float() @ w.float().t()) > 5e-3)
            dy = torch.randn(rows, N, device=dev, dtype=torch.bfloat16)
            dx, dyg = fc.all_gather_gemm_nn(dy, w, 'tp')
            bad += int(rel(dx, M.all_gather_dim0(dy, 'tp').float() @ w.float()) > 5e-3)
            xf = torch.randn(rows * world, K, device=dev, dtype=torch.bfloat16)
            yr = fc.gemm_reduce_scatter(xf, w, 'tp')
            bad += int(rel(yr, M.reduce_scatter_dim0(xf.float() @ w.float().t(), 'tp')) > 8e-3)
            if N % 64 == 0:
                dyf = torch.randn(rows * world, N, device=dev, dtype=torch.bfloat16)
                dxr = fc.gemm_reduce_scatter_nn(dyf, w, 'tp')
                bad += int(rel(dxr, M.reduce_scatter_dim0(dyf.float() @ w.float(), 'tp')) > 8e-3)
    torch.cuda.synchronize()
    _lib.check_status()
    t = torch.tensor([bad], device=dev)
    dist.all_reduce(t)
    assert t.item() == 0, f'{t.item()} fused-kernel mismatches'

    # end to end: one TP=2 + SP training step, fused vs library collectives, same seed
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    losses = {}
    for fused in ('1', '0'):
        os.environ['MCB200_FUSED_COMM'] = fused
        cfg = model_config('qwen3_tiny', bf16=True, tensor_model_parallel_size=world, sequence_parallel=True)
        tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=99))
        ds = SyntheticPackedDataset(1024, 1024, seg_lo=128, seg_hi=512, seed=5)
        mbs = [ds.next_microbatch() for _ in range(2)]
        losses[fused] = [tr.train_step(mbs) for _ in range(3)]
    torch.cuda.synchronize()
    _lib.check_status()
    for a, b in zip(losses['1'], losses['0']):
        assert abs(a - b) < 3e-2, losses
    if rank == 0:
        print('ALL OK', losses)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
