"""The command-line trainer: a short run on a tiny preset with token-file data, saving and resuming."""
import json
import os
import subprocess
import sys

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cli_trains_saves_and_resumes(tmp_path):
    tokens = np.random.default_rng(0).integers(0, 1024, size=20000, dtype=np.int32)
    data = str(tmp_path / 'tokens.npy')
    np.save(data, tokens)
    out = str(tmp_path / 'out')
    base = [sys.executable, '-m', 'mcore_bridge_b200.train.cli', '--model', 'qwen3_tiny', '--dtype', 'fp32', '--seq-len',
            '128', '--global-batch', '4', '--micro-batch-size', '2', '--data', data, '--lr', '1e-3', '--save', out]
    env = dict(os.environ, PYTHONPATH=REPO, CUDA_VISIBLE_DEVICES='')
    r = subprocess.run(base + ['--steps', '3'], env=env, capture_output=True, text=True, timeout=600, cwd=REPO)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [json.loads(l[l.index('{'):]) for l in (r.stdout + r.stderr).splitlines() if '"step"' in l]
    assert [l['step'] for l in lines] == [1, 2, 3] and all(l['loss'] == l['loss'] for l in lines)
    assert os.path.exists(os.path.join(out, 'model.safetensors'))
    assert os.path.isdir(os.path.join(out, 'state'))
    r = subprocess.run(base + ['--steps', '4', '--resume', os.path.join(out, 'state')], env=env, capture_output=True,
                       text=True, timeout=600, cwd=REPO)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [json.loads(l[l.index('{'):]) for l in (r.stdout + r.stderr).splitlines() if '"step"' in l]
    assert [l['step'] for l in lines] == [4]
    resumed = lines[0]
    # the resumed run continues the data stream: its step 4 is the step 4 of an uninterrupted run
    r = subprocess.run(base[:-2] + ['--steps', '4'], env=env, capture_output=True, text=True, timeout=600, cwd=REPO)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [json.loads(l[l.index('{'):]) for l in (r.stdout + r.stderr).splitlines() if '"step"' in l]
    assert lines[-1]['step'] == 4 and abs(lines[-1]['loss'] - resumed['loss']) < 1e-5, (lines[-1], resumed)


def test_cli_overrides_reach_the_model_config(tmp_path):
    from mcore_bridge_b200.train.cli import parse_overrides
    got = parse_overrides(['cp_comm_type=allgather', 'cpu-offloading=true', 'offload_modules=["core_attn", "mlp_norm"]',
                           'recompute_num_layers=2', "moe_router_dtype='fp32'"])
    assert got == {'cp_comm_type': 'allgather', 'cpu_offloading': True, 'offload_modules': ['core_attn', 'mlp_norm'],
                   'recompute_num_layers': 2, 'moe_router_dtype': 'fp32'}
    env = dict(os.environ, PYTHONPATH=REPO, CUDA_VISIBLE_DEVICES='')
    base = [sys.executable, '-m', 'mcore_bridge_b200.train.cli', '--model', 'qwen3_tiny', '--dtype', 'fp32', '--seq-len',
            '64', '--global-batch', '2', '--micro-batch-size', '1', '--steps', '1']
    r = subprocess.run(base + ['--set', 'fine_grained_activation_offloading=true', '--set',
                               'offload_modules=["core_attn"]'], env=env, capture_output=True, text=True, timeout=600,
                       cwd=REPO)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    r = subprocess.run(base + ['--set', 'no_such_field=1'], env=env, capture_output=True, text=True, timeout=600, cwd=REPO)
    assert r.returncode != 0 and 'no_such_field' in (r.stdout + r.stderr)
