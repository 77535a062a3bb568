"""Worker (torchrun, one process per GPU): the same tiny models trained for two optimizer steps under several parallel
layouts on real GPUs (NCCL, in-tree kernels, peer-memory collectives) must reproduce the data-parallel run of the same
global batch.  Weights travel through the Hugging Face checkpoint bridge, so every layout starts from the same values.
bf16 parameters: losses agree to bf16 rounding, not bit for bit."""
import os
import shutil
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch.distributed as dist
from mcore_bridge_b200.ops import _lib
from mcore_bridge_b200.parallel import state as ps

ps.init_distributed()
world, rank = dist.get_world_size(), dist.get_rank()
dev = torch.device('cuda', torch.cuda.current_device())
STEPS, GLOBAL_MB = 2, 4


def make_ckpt(name, hf_cls):
    from mcore_bridge_b200.train.presets import hf_config
    d = [None]
    if rank == 0:
        torch.manual_seed(0)
        hf = hf_cls(hf_config(name)).float()
        with torch.no_grad():
            for p in hf.parameters():
                p.normal_(0, 0.05) if p.dim() >= 2 else p.normal_(1.0, 0.05)
        d[0] = tempfile.mkdtemp(prefix='mcb200_layouts_')
        hf.save_pretrained(d[0])
    dist.broadcast_object_list(d, src=0)
    return d[0]


def run(name, ckpt, tp=1, pp=1, cp=1, ep=1, aux=0.0):
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                 context_parallel_size=cp, expert_model_parallel_size=ep)
    extra = dict(moe_aux_loss_coeff=aux) if aux else {}
    cfg = model_config(name, None, params_dtype=torch.bfloat16, bf16=True, tensor_model_parallel_size=tp,
                       pipeline_model_parallel_size=pp, context_parallel_size=cp, expert_model_parallel_size=ep,
                       sequence_parallel=tp > 1, **extra)
    tr = Trainer(cfg, TrainConfig(lr=1e-3, init_seed=None, clip_grad=1.0))
    cfg.bridge.load_weights(tr.models, ckpt)
    tr.optimizer = type(tr.optimizer)(tr.ddp, 1e-3, eps=1e-3, clip_grad=1.0)
    dp = ps.get_world_size('dp')
    dp_rank = ps.get_rank_in('dp') if dp > 1 else 0
    ds = SyntheticPackedDataset(1024, 1024, seg_lo=128, seg_hi=512, seed=3, pin=False, segment_multiple=4)
    losses = []
    for _ in range(STEPS):
        mbs = [ds.next_microbatch() for _ in range(GLOBAL_MB)]
        losses.append(float(tr.train_step(mbs[dp_rank::dp])))
    torch.cuda.synchronize()
    _lib.check_status()
    # only the last pipeline stage sees the loss: share it
    t = torch.tensor(losses if ps.is_pipeline_last_stage() else [0.0] * STEPS, device=dev, dtype=torch.float64)
    n = torch.tensor([1.0 if ps.is_pipeline_last_stage() else 0.0], device=dev, dtype=torch.float64)
    dist.all_reduce(t)
    dist.all_reduce(n)
    return (t / n).tolist()


def main():
    from transformers import Qwen3ForCausalLM, Qwen3MoeForCausalLM
    ok = True
    dense = make_ckpt('qwen3_tiny', Qwen3ForCausalLM)
    moe = make_ckpt('qwen3_moe_tiny', Qwen3MoeForCausalLM)
    base = run('qwen3_tiny', dense)                       # data parallel over all ranks
    base_moe = run('qwen3_moe_tiny', moe, aux=1e-2)
    layouts = [('tp2', 'qwen3_tiny', dict(tp=2)), ('pp2', 'qwen3_tiny', dict(pp=2)), ('cp2', 'qwen3_tiny', dict(cp=2)),
               ('ep2', 'qwen3_moe_tiny', dict(ep=2, aux=1e-2)), ('moe_pp2', 'qwen3_moe_tiny', dict(pp=2, aux=1e-2))]
    if world >= 4:
        layouts += [('tp2_pp2', 'qwen3_tiny', dict(tp=2, pp=2)), ('tp2_cp2', 'qwen3_tiny', dict(tp=2, cp=2)),
                    ('tp2_ep2', 'qwen3_moe_tiny', dict(tp=2, ep=2, aux=1e-2))]
    for tag, name, kw in layouts:
        ref = base if name == 'qwen3_tiny' else base_moe
        got = run(name, dense if name == 'qwen3_tiny' else moe, **kw)
        good = all(abs(a - b) < 2e-2 * max(1.0, abs(b)) for a, b in zip(got, ref))
        ok &= good
        if rank == 0:
            print(f'{tag}: losses {["%.4f" % v for v in got]} vs data-parallel {["%.4f" % v for v in ref]} '
                  f'{"OK" if good else "FAIL"}', flush=True)
    dist.barrier()
    if rank == 0:
        shutil.rmtree(dense, ignore_errors=True)
        shutil.rmtree(moe, ignore_errors=True)
        print('ALL OK' if ok else 'SOME FAILED', flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == '__main__':
    main()
