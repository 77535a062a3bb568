"""The benchmark script's contract pieces that need no GPU: the reference arm's one-line answer and the second stage of
the 8-GPU run (it must hand back the dense result even when the second model cannot run)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env=None):
    e = dict(os.environ)
    for k in ('RANK', 'WORLD_SIZE', 'LOCAL_RANK', 'MASTER_ADDR', 'MASTER_PORT'):
        e.pop(k, None)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, 'bench.py')] + args, capture_output=True, text=True,
                          env=e, timeout=600)


def test_reference_arm_prints_one_unavailable_line():
    res = _run(['--impl', 'reference', '--gpus', '1', '--steps', '2', '--warmup', '3'])
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out['impl'] == 'reference' and out['unavailable']


def test_second_stage_keeps_the_dense_result_when_the_moe_run_fails(tmp_path):
    """Without a GPU the second stage cannot even select a device: it must still print the first stage's result, with
    the failure recorded under ``secondary``, and exit 0."""
    import socket
    with socket.socket() as sk:
        sk.bind(('127.0.0.1', 0))
        port = sk.getsockname()[1]
    dense = {'metric': 'train tokens/s', 'value': 1.0, 'n_gpus': 8, 'selfcheck_failed': []}
    path = tmp_path / 'stage1.json'
    path.write_text(json.dumps({'port': port, 'result': dense}))
    res = _run(['--gpus', '8', '--stage2', str(path)],
               env={'RANK': '0', 'WORLD_SIZE': '1', 'LOCAL_RANK': '0', 'MASTER_ADDR': '127.0.0.1',
                    'MASTER_PORT': str(port), 'CUDA_VISIBLE_DEVICES': ''})
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip().startswith('{')]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out['value'] == 1.0 and out['n_gpus'] == 8
    assert out['secondary']['model'] == 'qwen3_30b_a3b' and 'error' in out['secondary']
    assert not path.exists()
