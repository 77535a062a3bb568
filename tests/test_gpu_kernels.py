"""Numerics of every in-tree CUDA kernel against a plain PyTorch fp32 reference of the same op (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()


@pytest.fixture(autouse=True)
def _status():
    from mcore_bridge_b200.ops import _lib
    assert _lib.available(), 'the CUDA library must load on a GPU box'
    yield
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize('M,N,K', [(128, 256, 64), (384, 512, 256), (1000, 776, 520), (2048, 4096, 1024), (100, 72, 40)])
@pytest.mark.parametrize('bn', [0, 256, 128, 64])
def test_gemm_nt(M, N, K, bn):
    from mcore_bridge_b200.ops import gemm
    torch.manual_seed(0)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    ref = x.float() @ w.float().t()
    assert rel(gemm.mm_nt(x, w, force_bn=bn), ref) < 5e-3
    assert rel(gemm.mm_nt(x, w, bias=b, force_bn=bn), ref + b.float()) < 5e-3
    assert rel(gemm.mm_nt(x, w, out_dtype=torch.float32, force_bn=bn), ref) < 1e-5


@pytest.mark.parametrize('M,N,K', [(128, 256, 64), (1000, 776, 520), (2048, 1024, 4096), (264, 136, 1096)])
def test_gemm_nn_tn(M, N, K):
    from mcore_bridge_b200.ops import gemm
    torch.manual_seed(1)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    assert rel(gemm.mm_nn(dy, w), dy.float() @ w.float()) < 5e-3
    ref = dy.float().t() @ x.float()
    assert rel(gemm.mm_tn(dy, x, out_dtype=torch.float32), ref) < 1e-4
    acc = torch.ones(N, K, device=DEV, dtype=torch.float32)
    gemm.mm_tn(dy, x, out=acc, accumulate=True)
    assert rel(acc, ref + 1) < 1e-4


def test_grouped_gemm():
    from mcore_bridge_b200.ops import gemm
    torch.manual_seed(2)
    G, N, K = 8, 512, 1024
    counts = torch.tensor([300, 0, 128, 77, 513, 1, 256, 1000])
    padded = (counts + 127) // 128 * 128
    off = torch.zeros(G + 1, dtype=torch.int32)
    off[1:] = padded.cumsum(0)
    R = int(off[-1]) + 256
    x = torch.zeros(R, K, device=DEV, dtype=torch.bfloat16)
    dy = torch.zeros(R, N, device=DEV, dtype=torch.bfloat16)
    for g in range(G):
        x[off[g]:off[g] + counts[g]] = torch.randn(int(counts[g]), K, device=DEV, dtype=torch.bfloat16)
        dy[off[g]:off[g] + counts[g]] = torch.randn(int(counts[g]), N, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(G, N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    offd = off.to(DEV)
    end = int(off[-1])
    y = gemm.grouped_mm_nt(x, w, offd)
    dx = gemm.grouped_mm_nn(dy, w, offd)
    dw = gemm.grouped_mm_tn(dy, x, offd, out_dtype=torch.float32)
    for g in range(G):
        s, e = int(off[g]), int(off[g + 1])
        if e > s:
            assert rel(y[s:e], x[s:e].float() @ w[g].float().t()) < 5e-3
            assert rel(dx[s:e], dy[s:e].float() @ w[g].float()) < 5e-3
        assert (dw[g] - dy[s:e].float().t() @ x[s:e].float()).abs().max() < 1e-2 * max(1.0, float(counts[g])) ** 0.5
    assert end <= R


@pytest.mark.parametrize('H', [128, 256, 4096, 7168])
@pytest.mark.parametrize('zc', [False, True])
def test_rmsnorm(H, zc):
    from mcore_bridge_b200.ops import norm
    torch.manual_seed(3)
    x = torch.randn(1000, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(H, device=DEV) * 0.1 + (0 if zc else 1)).to(torch.bfloat16).requires_grad_()
    y = norm.rmsnorm(x, w, 1e-6, zc)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = norm.rmsnorm_ref(xr, wr, 1e-6, zc)
    yr.backward(g.float())
    assert rel(y, yr) < 5e-3 and rel(x.grad, xr.grad) < 1e-2 and rel(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize('kind,clamp,off', [('swiglu', 0, 0), ('quick_geglu', 7.0, 1.0), ('geglu_tanh', 0, 0)])
def test_glu(kind, clamp, off):
    from mcore_bridge_b200.ops import activation
    torch.manual_seed(4)
    x = torch.randn(777, 2 * 1536, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    pr = torch.rand(777, device=DEV, requires_grad=True)
    y = activation.glu(x, kind, pr, clamp, off)
    g = torch.randn_like(y)
    y.backward(g)
    xr, prr = x.detach().float().requires_grad_(), pr.detach().clone().requires_grad_()
    yr = activation.glu_ref(xr, kind, prr, clamp, off)
    yr.backward(g.float())
    assert rel(y, yr) < 5e-3 and rel(x.grad, xr.grad) < 1e-2 and rel(pr.grad, prr.grad) < 1e-2


@pytest.mark.parametrize('ng,qpg,d,gate,rotf,inter,nrm', [(2, 4, 128, False, 1.0, False, True), (1, 8, 256, True, 0.25, False, True),
                                                          (4, 1, 64, False, 1.0, True, False), (2, 2, 128, False, 0.0, False, True)])
def test_qkv_split_norm_rope(ng, qpg, d, gate, rotf, inter, nrm):
    from mcore_bridge_b200.ops import rope
    torch.manual_seed(5)
    T = 515
    ld = ng * (qpg * (2 if gate else 1) + 2) * d
    qkv = torch.randn(T, ld, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    wq = (torch.randn(d, device=DEV) * 0.1 + 1).to(torch.bfloat16).requires_grad_() if nrm else None
    wk = (torch.randn(d, device=DEV) * 0.1 + 1).to(torch.bfloat16).requires_grad_() if nrm else None
    rot = int(d * rotf)
    cos = sin = None
    if rot:
        ang = torch.rand(T, rot // 2, device=DEV) * 6.28
        cos, sin = ang.cos(), ang.sin()
    outs = rope.qkv_split_norm_rope(qkv, wq, wk, cos, sin, ng, qpg, d, gate, inter, 1e-6, False)
    gs = [torch.randn_like(o) if o is not None else None for o in outs]
    torch.autograd.backward([o for o in outs if o is not None], [g for g in gs if g is not None])
    qr = qkv.detach().float().requires_grad_()
    wqr = wq.detach().float().requires_grad_() if nrm else None
    wkr = wk.detach().float().requires_grad_() if nrm else None
    outr = rope.qkv_split_norm_rope_ref(qr, wqr, wkr, cos, sin, ng, qpg, d, gate, inter, 1e-6, False)
    torch.autograd.backward([o for o in outr if o is not None], [g.float() for g in gs if g is not None])
    for a, b in zip(outs, outr):
        if a is not None:
            assert rel(a, b) < 5e-3
    assert rel(qkv.grad, qr.grad) < 1e-2
    if nrm:
        assert rel(wq.grad, wqr.grad) < 1e-2 and rel(wk.grad, wkr.grad) < 1e-2


@pytest.mark.parametrize('V', [1000, 1024, 32000])
def test_fused_linear_cross_entropy(V):
    from mcore_bridge_b200.ops import cross_entropy
    torch.manual_seed(6)
    T = 300
    h = torch.randn(T, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, 512, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    lab = torch.randint(0, V, (T,), device=DEV)
    loss = cross_entropy.fused_linear_cross_entropy(h, w, lab, 'tp', chunk=128)
    gl = torch.rand(T, device=DEV)
    loss.backward(gl)
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr_ = torch.nn.functional.cross_entropy(hr @ wr.t(), lab, reduction='none')
    lr_.backward(gl)
    assert rel(loss, lr_) < 1e-3 and rel(h.grad, hr.grad) < 1e-2 and rel(w.grad, wr.grad) < 1e-2
    # a vocabulary shard that starts at a non-zero column: the epilogue statistics against the torch ones
    start = 512
    glob = lab + start - (V // 2)                      # some labels fall outside this shard on either side
    m, s, t = cross_entropy._head_stats(h.detach(), w.detach(), glob, start)
    mr, sr, tr = cross_entropy._stats_torch(h.detach().float() @ w.detach().float().t(), glob, start)
    assert rel(m, mr) < 1e-3 and rel(m + torch.log(s), mr + torch.log(sr)) < 1e-3 and (t - tr).abs().max() < 2e-2


def test_fused_adam_matches_torch():
    from mcore_bridge_b200.train.distributed_optimizer import DistributedDataParallel, DistributedOptimizer
    torch.manual_seed(7)
    lin = torch.nn.Linear(256, 512, bias=True).to(DEV).to(torch.bfloat16)
    ref = torch.nn.Linear(256, 512, bias=True).to(DEV).float()
    ref.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})
    ddp = DistributedDataParallel(lin)
    opt = DistributedOptimizer([ddp], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=0.0)
    ropt = torch.optim.AdamW([{'params': [ref.weight], 'weight_decay': 0.1}, {'params': [ref.bias], 'weight_decay': 0.0}],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for step in range(3):
        gw = torch.randn(512, 256, device=DEV)
        gb = torch.randn(512, device=DEV)
        opt.zero_grad()
        lin.weight.main_grad.copy_(gw)
        lin.bias.main_grad.copy_(gb)
        ref.weight.grad, ref.bias.grad = gw.clone(), gb.clone()
        opt.step()
        ropt.step()
    assert rel(lin.weight, ref.weight) < 5e-3 and rel(lin.bias, ref.bias) < 5e-3
    main_w = [s[3] for s in opt.shards]
    assert any(rel(m[:ref.weight.numel()].view_as(ref.weight), ref.weight) < 1e-5 for m in main_w if m.numel() >= ref.weight.numel())


def test_train_step_tiny_model_loss_goes_down():
    from mcore_bridge_b200.ops import _lib
    from mcore_bridge_b200.train.data import SyntheticPackedDataset
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import TrainConfig, Trainer
    cfg = model_config('qwen3_tiny', bf16=True, recompute_granularity='full', recompute_method='uniform',
                       recompute_num_layers=1)
    tr = Trainer(cfg, TrainConfig(lr=2e-3))
    ds = SyntheticPackedDataset(1024, 1024, seg_lo=128, seg_hi=512, seed=5)
    mbs = [ds.next_microbatch() for _ in range(2)]
    before = _lib.LAUNCHES
    losses = [tr.train_step(mbs) for _ in range(8)]
    assert _lib.LAUNCHES > before
    assert losses[-1] < losses[0] - 0.3, losses


def test_bf16_model_matches_fp32_reference_model():
    """Whole-model check: the CUDA path (bf16) against the same weights run through the torch fp32 path."""
    from mcore_bridge_b200 import ModelConfig, get_mcore_model, hf_to_mcore_config
    from mcore_bridge_b200.train.presets import hf_config
    from mcore_bridge_b200.train.trainer import init_weights
    kw = hf_to_mcore_config(hf_config('qwen3_tiny'))
    cfg = ModelConfig(**kw, bf16=True)
    model = get_mcore_model(cfg)[0]
    init_weights(model, 0.05, 11)
    cfg32 = ModelConfig(**kw, params_dtype=torch.float32)
    ref = get_mcore_model(cfg32)[0]
    ref.load_state_dict({k: v.float() for k, v in model.state_dict().items()})
    ids = torch.randint(0, 1024, (2, 256), device=DEV)
    labels = torch.randint(0, 1024, (2, 256), device=DEV)
    loss = model(ids, labels=labels).mean()
    loss_ref = ref(ids, labels=labels).mean()
    assert abs(loss.item() - loss_ref.item()) < 3e-2
    loss.backward()
    loss_ref.backward()
    g, gr = model.decoder.layers[0].mlp.linear_fc1.weight.grad, ref.decoder.layers[0].mlp.linear_fc1.weight.grad
    assert rel(g, gr) < 5e-2


@pytest.mark.parametrize('T,nq,nkv,d,segs', [(256, 2, 1, 128, [256]), (300, 4, 2, 128, [100, 200]),
                                             (1000, 4, 4, 64, [77, 500, 423]), (1536, 4, 1, 128, [512, 1, 1023]),
                                             (2048, 8, 2, 128, [700, 1348]),
                                             # T not a multiple of the 128-row tile together with 8 query heads per kv head
                                             (1100, 8, 1, 128, [333, 767])])
def test_attention_kernels(T, nq, nkv, d, segs):
    """Forward (two-pass softmax) and backward (delta, dQ, dK/dV kernels) against fp32 masked-softmax attention."""
    from mcore_bridge_b200.ops import attention as A
    from mcore_bridge_b200.ops import attention_cuda as AC
    torch.manual_seed(8)
    q = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(segs).cumsum(0)), dtype=torch.int32, device=DEV)
    assert AC.supported(q, k, v, True, None, None, None)
    from mcore_bridge_b200.ops import _lib
    assert hasattr(_lib.lib(), 'mcb_attn_bwd')
    q2, k2, v2 = (t.clone().requires_grad_() for t in (q, k, v))
    o = AC.attention(q2, k2, v2, cu, max(segs), None)
    g = torch.randn_like(o)
    o.backward(g)
    qr, kr, vr = (t.float().clone().requires_grad_() for t in (q, k, v))
    ref = A.attention_ref(qr, kr, vr, cu, cu)
    ref.backward(g.float())
    assert rel(o, ref) < 1e-2
    assert rel(q2.grad, qr.grad) < 2e-2 and rel(k2.grad, kr.grad) < 2e-2 and rel(v2.grad, vr.grad) < 2e-2


@pytest.mark.parametrize('E,k,sig,groups', [(8 * 4, 2, False, None), (128, 8, False, None), (64, 6, True, 8), (256, 8, True, 8)])
def test_router_kernel_matches_torch(E, k, sig, groups):
    from mcore_bridge_b200.layers import moe_fused as F
    from mcore_bridge_b200.ops import moe as moe_ops
    torch.manual_seed(9)
    T = 777
    logits = torch.randn(T, E, device=DEV) * 2
    bias = torch.randn(E, device=DEV) * 0.1 if sig else None
    gt = 4 if groups else None
    assert F.router_supported(E, k, groups)
    lg = logits.clone().requires_grad_()
    probs_out = torch.empty(T, k, device=DEV)
    idx_out = torch.empty(T, k, dtype=torch.int32, device=DEV)
    counts = torch.empty(E, dtype=torch.int32, device=DEV)
    renorm = True
    probs, idx, ssum = F._RouterFn.apply(lg, bias, None, k, sig, renorm, groups, gt, 2.5, probs_out, idx_out, counts)
    lr = logits.clone().requires_grad_()
    p_ref, i_ref, s_ref = moe_ops.topk_routing(lr, k, 'sigmoid' if sig else 'softmax', False, groups, gt, 2.5, bias)
    # same experts (order inside the k may differ on ties: compare as sets through a scatter)
    dense = torch.zeros(T, E, device=DEV).scatter_(1, idx.long(), probs)
    dense_ref = torch.zeros(T, E, device=DEV).scatter_(1, i_ref, p_ref)
    assert rel(dense, dense_ref) < 1e-4
    assert torch.equal(counts.long(), torch.bincount(i_ref.reshape(-1), minlength=E))
    assert rel(ssum, s_ref.sum(0)) < 1e-4
    w = torch.randn(T, E, device=DEV)
    v = torch.randn(E, device=DEV)
    ((dense * w).sum() + (ssum * v).sum()).backward()
    ((dense_ref * w).sum() + (s_ref.sum(0) * v).sum()).backward()
    assert rel(lg.grad, lr.grad) < 1e-3


@pytest.mark.parametrize('M,N,K', [(256, 256, 512), (1000, 384, 1024), (4096, 2048, 7168)])
def test_fp8_blockscaled_gemm_and_quant(M, N, K):
    """Quantisation kernels equal the torch restatement bit for bit; the GEMM equals the fp32 product of the
    dequantised operands."""
    from mcore_bridge_b200.ops import fp8
    torch.manual_seed(11)
    x = (torch.randn(M, K, device=DEV) * torch.rand(M, 1, device=DEV) * 3).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    x8, sx = fp8.quantize_1x128(x)
    x8r, sxr = fp8.quantize_1x128_ref(x)
    assert torch.equal(sx, sxr)
    assert (x8.float() - x8r.float()).abs().max().item() == 0
    w8, sw, w8t, swt = fp8.quantize_128x128(w, with_transpose=True)
    w8r, swr = fp8.quantize_128x128_ref(w)
    assert torch.equal(sw, swr) and torch.equal(swt, swr.t())
    assert (w8.float() - w8r.float()).abs().max().item() == 0
    assert torch.equal(w8t.view(torch.uint8), w8.view(torch.uint8).t())
    c = fp8.gemm_blockscaled(x8, sx, w8, sw)
    ref = fp8.gemm_blockscaled_ref(x8, sx, w8, sw, out_dtype=torch.float32)
    assert rel(c, ref) < 5e-3
    # against the unquantised product: fp8 rounding only
    assert rel(c, x.float() @ w.float().t()) < 6e-2


def test_fp8_linear_forward_backward():
    from mcore_bridge_b200.ops.linear import LinearSpec, linear
    torch.manual_seed(12)
    x = torch.randn(512, 1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(768, 1024, device=DEV) * 0.03).to(torch.bfloat16).requires_grad_()
    y = linear(x, w, None, LinearSpec(fp8=True))
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    assert rel(y, yr) < 6e-2 and rel(x.grad, xr.grad) < 6e-2 and rel(w.grad, wr.grad) < 2e-2


def test_linear_attention_elementwise_kernels():
    """Causal conv1d+SiLU and gated RMSNorm kernels (forward and backward) against the torch restatements."""
    from mcore_bridge_b200.ops import gdn as G
    torch.manual_seed(13)
    T, C, K = 700, 256, 4
    cu = torch.tensor([0, 100, 101, 450, 700], dtype=torch.int32, device=DEV)
    x = torch.randn(T, C, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(C, K, device=DEV) * 0.5).to(torch.bfloat16)
    g = torch.randn(T, C, device=DEV, dtype=torch.bfloat16)
    x1, w1 = x.clone().requires_grad_(), w.clone().requires_grad_()
    y = G.causal_conv1d_silu(x1, w1, None, cu)
    y.backward(g)
    x2, w2 = x.float().requires_grad_(), w.float().requires_grad_()
    yr = G._causal_conv1d_silu_torch(x2, w2, None, cu)
    yr.backward(g.float())
    assert rel(y, yr) < 1e-2 and rel(x1.grad, x2.grad) < 1e-2 and rel(w1.grad, w2.grad) < 1e-2
    rows, D = 3000, 128
    a = torch.randn(rows, D, device=DEV, dtype=torch.bfloat16)
    z = torch.randn(rows, D, device=DEV, dtype=torch.bfloat16)
    wn = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16)
    gg = torch.randn(rows, D, device=DEV, dtype=torch.bfloat16)
    a1, z1, n1 = a.clone().requires_grad_(), z.clone().requires_grad_(), wn.clone().requires_grad_()
    o = G.gated_rmsnorm(a1, z1, n1, 1e-6)
    o.backward(gg)
    a2, z2, n2 = a.float().requires_grad_(), z.float().requires_grad_(), wn.float().requires_grad_()
    orf = G._gated_rmsnorm_torch(a2, z2, n2, 1e-6)
    orf.backward(gg.float())
    assert rel(o, orf) < 1e-2 and rel(a1.grad, a2.grad) < 1.5e-2 and rel(z1.grad, z2.grad) < 1e-2
    assert rel(n1.grad, n2.grad) < 1e-2


@pytest.mark.parametrize('d', [64, 128])
def test_simple_gla_kernels(d):
    """Recurrent lightning-attention kernels against the masked-decay matmul form, packed sequences."""
    from mcore_bridge_b200.ops import gdn as G
    torch.manual_seed(14)
    T, h = 600, 4
    cu = torch.tensor([0, 256, 257, 600], dtype=torch.int32, device=DEV)
    q, k, v = (torch.randn(T, h, d, device=DEV, dtype=torch.bfloat16) * 0.5 for _ in range(3))
    decay = -torch.rand(h, device=DEV) * 0.2 - 0.01
    g = torch.randn(T, h, d, device=DEV, dtype=torch.bfloat16)
    q1, k1, v1 = (t.clone().requires_grad_() for t in (q, k, v))
    o = G.simple_gla(q1, k1, v1, decay, cu)
    o.backward(g)
    q2, k2, v2 = (t.float().requires_grad_() for t in (q, k, v))
    orf = G.simple_gla_ref(q2, k2, v2, decay, cu)
    orf.backward(g.float())
    assert rel(o, orf) < 1e-2
    assert rel(q1.grad, q2.grad) < 1e-2 and rel(k1.grad, k2.grad) < 1e-2 and rel(v1.grad, v2.grad) < 1e-2


def test_lean_activation_blocks_match_unfused():
    """norm_linear / glu_linear (recompute in backward) give the same loss and gradients as the unfused layers."""
    from mcore_bridge_b200 import get_mcore_model
    from mcore_bridge_b200.train.presets import model_config
    from mcore_bridge_b200.train.trainer import init_weights
    ids = torch.randint(0, 1024, (2, 256), device=DEV, generator=torch.Generator(device=DEV).manual_seed(3))
    labels = torch.randint(0, 1024, (2, 256), device=DEV, generator=torch.Generator(device=DEV).manual_seed(4))
    out = {}
    for lean in (True, False):
        cfg = model_config('qwen3_tiny', bf16=True, lean_activations=lean)
        model = get_mcore_model(cfg)[0]
        init_weights(model, 0.02, 7)
        loss = model(ids, labels=labels).mean()
        loss.backward()
        layer = model.decoder.layers[1]
        out[lean] = (loss.detach(), layer.mlp.linear_fc1.weight.grad.clone(), layer.mlp.linear_fc2.weight.grad.clone(),
                     layer.mlp.linear_fc1.layer_norm_weight.grad.clone(),
                     layer.self_attention.linear_qkv.weight.grad.clone(),
                     model.embedding.word_embeddings.weight.grad.clone())
    assert torch.equal(out[True][0], out[False][0])
    for a, b in zip(out[True][1:], out[False][1:]):
        assert rel(a, b) < 1e-3


@pytest.mark.parametrize('T,H,segs,k', [(512, 4, [512], 64), (1000, 8, [300, 700], 128), (2048, 64, [2048], 512)])
def test_dsa_indexer_scores_and_topk(T, H, segs, k):
    """tcgen05 lightning-indexer scores against the fp32 einsum; radix-select top-k against torch.topk (as sets, and
    by the selected values since ties may resolve differently)."""
    from mcore_bridge_b200.ops import dsa
    from mcore_bridge_b200.ops.attention_cuda import seq_start_from_cu
    torch.manual_seed(21)
    q = torch.randn(T, H, 128, device=DEV, dtype=torch.bfloat16)
    kk = torch.randn(T, 128, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(T, H, device=DEV) * 0.1
    cu = torch.tensor([0] + list(torch.tensor(segs).cumsum(0)), dtype=torch.int32, device=DEV)
    ss = seq_start_from_cu(cu, T, q.device)
    pos = torch.arange(T, device=DEV)
    mask = (ss[:, None] <= pos[None, :]) & (pos[None, :] <= pos[:, None])
    ref = dsa.index_scores(q, kk, w, mask)
    got = dsa.index_scores_cuda(q, kk, w, ss)
    assert torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = ~torch.isinf(ref)
    assert ((got[fin] - ref[fin]).abs().max() / ref[fin].abs().max()).item() < 2e-2
    idx = dsa.topk_indices(got, k)
    assert idx.shape == (T, k)
    vals = got.gather(1, idx).sort(dim=1, descending=True).values
    want = got.topk(k, dim=1).values
    assert torch.equal(vals, want)
    # no position is selected twice
    assert (idx.sort(dim=1).values[:, 1:] != idx.sort(dim=1).values[:, :-1]).all()


def test_bounded_wait_reports_status_and_context_survives():
    """A device wait on a flag that nothing sets runs out after its (shortened) limit, the kernel returns with the
    peer-flag status code, the host check raises, and the context is still usable for the next kernel."""
    import ctypes

    from mcore_bridge_b200.ops import _lib, gemm
    dev = torch.device('cuda', torch.cuda.current_device())
    status = _lib.status_word(dev)
    torch.cuda.synchronize()
    old_limit = int(status[1].item())
    flags = torch.zeros(64, dtype=torch.int32, device=dev)       # flag slot 0 stays 0, the wait wants 1
    ptrs = (ctypes.c_void_p * 1)(flags.data_ptr())
    try:
        status[1] = 50                                            # milliseconds
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = _lib.lib().mcb_flag_wait(ptrs, ctypes.c_int(1), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_uint(1),
                                      _lib.ptr(status), _lib.stream_ptr())
        t1.record()
        assert rc == 0
        torch.cuda.synchronize()
        assert 30.0 < t0.elapsed_time(t1) < 2000.0                # gave up near the limit, not at the 10 s default
        assert int(status[0].item()) == 5
        with pytest.raises(_lib.KernelError, match='peer flag'):
            _lib.check_status(dev)
        assert int(status[0].item()) == 0                         # cleared by the check
    finally:
        status[1] = old_limit
        status[0] = 0
    x = torch.randn(256, 128, device=dev, dtype=torch.bfloat16)
    w = torch.randn(256, 128, device=dev, dtype=torch.bfloat16)
    assert rel(gemm.mm_nt(x, w), x.float() @ w.float().t()) < 5e-3


@pytest.mark.parametrize('M,N,K', [(512, 256, 128), (1000, 776, 520), (2048, 4096, 1024), (4096, 6144, 4096),
                                   (8192, 1024, 256)])
def test_gemm_cta_pair(M, N, K):
    """The 256 x 256 CTA-pair kernel (``force_bn=512``) in the three layouts of a linear layer, against fp32 matmuls
    and against the single-CTA kernel; a wrong 128-row half or 128-column half would show in the per-row check."""
    from mcore_bridge_b200.ops import gemm
    torch.manual_seed(3)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)

    def close(a, ref, tol):
        a, ref = a.float(), ref.float()
        assert rel(a, ref) < tol
        assert ((a - ref).norm(dim=-1).max() / ref.norm(dim=-1).mean()).item() < 4 * tol

    ref = x.float() @ w.float().t()
    close(gemm.mm_nt(x, w, force_bn=512), ref, 5e-3)
    close(gemm.mm_nt(x, w, bias=b, force_bn=512), ref + b.float(), 5e-3)
    close(gemm.mm_nt(x, w, out_dtype=torch.float32, force_bn=512), ref, 1e-5)
    close(gemm.mm_nn(dy, w, force_bn=512), dy.float() @ w.float(), 5e-3)
    acc = torch.randn(N, K, device=DEV, dtype=torch.float32)
    ref_tn = acc + dy.float().t() @ x.float()
    close(gemm.mm_tn(dy, x, out=acc, accumulate=True, force_bn=512), ref_tn, 1e-5)


@pytest.mark.parametrize('d,nq,nkv', [(128, 8, 2), (64, 4, 4)])
@pytest.mark.parametrize('cp', [2, 4])
def test_attention_ranges_context_parallel_layout(d, nq, nkv, cp):
    """The per-query key-range kernels on the zig-zag layout of every context-parallel rank (emulated on one GPU):
    output and all gradients against the masked-softmax reference on the whole stream."""
    from mcore_bridge_b200.ops import attention_cuda as ac
    from mcore_bridge_b200.ops.attention import attention_ref
    from mcore_bridge_b200.parallel.context_parallel import compute_layout
    torch.manual_seed(4)
    lens = [8 * cp * 20, 8 * cp * 3, 8 * cp * 41, 8 * cp * 7]           # multiples of 2 * cp, tiles straddle sequences
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    q = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16)
    do = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    ref = attention_ref(qr, kr, vr, cu, cu)
    for rank in range(cp):
        lay = compute_layout(cu, T // cp, cp, rank, torch.device(DEV))
        assert torch.equal(lay.scatter_index[lay.gather_index], torch.arange(T, device=DEV))
        ql = q[lay.q_stream].clone().requires_grad_()
        kf, vf = k.clone().requires_grad_(), v.clone().requires_grad_()
        o, lse = ac.attention_ranges(ql, kf, vf, lay.k_lo, lay.k_hi, lay.q_lo, lay.q_hi)
        assert rel(o, ref[lay.q_stream]) < 2e-2
        o.backward(do[lay.q_stream])
        gq, gk, gv = torch.autograd.grad(ref[lay.q_stream], (qr, kr, vr), do[lay.q_stream].float(), retain_graph=True)
        assert rel(ql.grad, gq[lay.q_stream]) < 3e-2
        assert rel(kf.grad, gk) < 3e-2 and rel(vf.grad, gv) < 3e-2
        worst = ((kf.grad.float() - gk).flatten(1).norm(dim=1).max() / gk.flatten(1).norm(dim=1).mean()).item()
        assert worst < 0.15, worst


def test_attention_ranges_bidirectional_and_empty_rows():
    """Non-causal packed attention (every query sees its whole sequence) and queries that see nothing."""
    from mcore_bridge_b200.ops import attention_cuda as ac
    from mcore_bridge_b200.ops.attention import attention_ref
    torch.manual_seed(5)
    lens = [300, 77, 513, 134]
    T, nq, nkv, d = sum(lens), 4, 2, 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    seg = torch.searchsorted(cu[1:].long().contiguous(), torch.arange(T, device=DEV), right=True)
    k_lo = cu[:-1][seg].to(torch.int32)
    k_hi = (cu[1:][seg] - 1).to(torch.int32)
    q_lo, q_hi = k_lo.clone(), k_hi.clone()
    # the queries of the second sequence see nothing
    dead = seg == 1
    k_lo[dead], k_hi[dead] = 1, 0
    q_lo[dead], q_hi[dead] = 1, 0
    q = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    do = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    o, lse = ac.attention_ranges(q, k, v, k_lo, k_hi, q_lo, q_hi)
    o.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_ref(qr, kr, vr, cu, cu, causal=False)
    live = ~dead
    assert rel(o[live], ref[live]) < 2e-2
    assert o[dead].abs().max().item() == 0.0 and torch.isinf(lse[:, dead]).all()
    (ref[live] * do[live].float()).sum().backward()
    assert rel(q.grad[live], qr.grad[live]) < 3e-2 and q.grad[dead].abs().max().item() == 0.0
    assert rel(k.grad, kr.grad) < 3e-2 and rel(v.grad, vr.grad) < 3e-2
    assert torch.isfinite(k.grad.float()).all() and torch.isfinite(q.grad.float()).all()


@pytest.mark.parametrize('d,nq,nkv', [(64, 8, 2), (128, 4, 4)])
@pytest.mark.parametrize('window,use_sinks', [(96, False), (None, True), (200, True)])
def test_attention_window_and_sinks(d, nq, nkv, window, use_sinks):
    """Sliding-window attention and learnable softmax sinks on the in-tree kernels (the GPT-OSS configuration), packed
    sequences, output and every gradient (the sinks' included) against the masked-softmax reference."""
    from mcore_bridge_b200.ops.attention import attention, attention_ref
    torch.manual_seed(8)
    lens = [333, 40, 700, 129]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    q = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    sinks = (torch.randn(nq, device=DEV) * 2).requires_grad_() if use_sinks else None
    do = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    w = None if window is None else (window, 0)
    o = attention(q, k, v, cu, max(lens), True, None, w, sinks)
    o.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    sr = sinks.detach().clone().requires_grad_() if use_sinks else None
    ref = attention_ref(qr, kr, vr, cu, cu, True, None, w, sr)
    ref.backward(do.float())
    assert rel(o, ref) < 2e-2
    assert rel(q.grad, qr.grad) < 3e-2 and rel(k.grad, kr.grad) < 3e-2 and rel(v.grad, vr.grad) < 3e-2
    if use_sinks:
        assert rel(sinks.grad, sr.grad) < 3e-2


def test_router_gate_on_tensor_cores_matches_fp32_linear():
    """Router logits and their gradients from the bf16 tensor-core GEMM (fp32 accumulate, two-term split of the fp32
    logit gradient) against the fp32 ``F.linear`` the router's fp32 mode describes."""
    from mcore_bridge_b200.layers.moe import _RouterGateFn
    torch.manual_seed(3)
    T, H, E = 1000, 512, 128
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(E, H, device=DEV) * 0.1).to(torch.bfloat16).requires_grad_()
    dl = torch.randn(T, E, device=DEV, dtype=torch.float32)
    y = _RouterGateFn.apply(x, w, torch.float32)
    y.backward(dl)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(dl)
    assert y.dtype == torch.float32
    assert (y - yr).abs().max().item() < 1e-3 * yr.abs().max().item()
    assert rel(x.grad, xr.grad) < 5e-3            # bf16 rounding of the result only
    assert rel(w.grad, wr.grad) < 5e-3
    # the split keeps the fp32 gradient's low bits: much closer than rounding dl to bf16 would be
    dx_fp32 = (dl.double() @ w.detach().double())
    hi_only = (dl.to(torch.bfloat16).double() @ w.detach().double())
    from mcore_bridge_b200.ops import gemm
    hi = dl.to(torch.bfloat16)
    d2 = torch.cat([hi, (dl - hi.float()).to(torch.bfloat16)], dim=1)
    dx_split = gemm.mm_nn(d2, torch.cat([w.detach(), w.detach()], 0), out_dtype=torch.float32)
    assert (dx_split.double() - dx_fp32).norm() < 0.05 * (hi_only - dx_fp32).norm()


def test_router_kernel_padding_mask_keeps_padded_tokens_out_of_the_statistics():
    """Padded tokens are routed like the others (probabilities and indices unchanged) but are not counted: the
    per-expert token counts and score sums cover the valid tokens only."""
    from mcore_bridge_b200.layers import moe_fused as F
    torch.manual_seed(10)
    T, E, k = 600, 64, 4
    logits = torch.randn(T, E, device=DEV) * 2
    valid = (torch.rand(T, device=DEV) > 0.2)
    out = {}
    for name, v in (('all', None), ('masked', valid.to(torch.uint8))):
        probs_out = torch.empty(T, k, device=DEV)
        idx_out = torch.empty(T, k, dtype=torch.int32, device=DEV)
        counts = torch.empty(E, dtype=torch.int32, device=DEV)
        probs, idx, ssum = F._RouterFn.apply(logits.clone(), None, v, k, False, True, None, None, 1.0, probs_out, idx_out,
                                             counts)
        out[name] = (probs.clone(), idx.clone(), ssum.clone(), counts.clone())
    assert torch.equal(out['all'][1], out['masked'][1]) and torch.equal(out['all'][0], out['masked'][0])
    ref_counts = torch.bincount(out['all'][1][valid].reshape(-1).long(), minlength=E)
    assert torch.equal(out['masked'][3].long(), ref_counts)
    ref_sum = torch.softmax(logits, dim=-1)[valid].sum(0)
    assert rel(out['masked'][2], ref_sum) < 1e-4


@pytest.mark.parametrize('cp', [2, 4])
def test_ring_attention_steps_on_the_kernels(cp):
    """The ring form of context-parallel attention with the ranks emulated on one GPU: per source rank one forward
    launch over a contiguous key range of that rank's tokens, partial results merged through their log-sum-exp; the
    backward launches get the final log-sum-exp and delta.  Output, dQ and the summed dK / dV against the reference."""
    from mcore_bridge_b200.ops import attention_cuda as ac
    from mcore_bridge_b200.ops.attention import attention_ref
    from mcore_bridge_b200.parallel.context_parallel import compute_layout
    torch.manual_seed(6)
    nq, nkv, d = 4, 2, 128
    lens = [8 * cp * 20, 8 * cp * 3, 8 * cp * 33]
    T = sum(lens)
    tl = T // cp
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    q = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(T, nkv, d, device=DEV, dtype=torch.bfloat16)
    do = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    ref = attention_ref(qr, kr, vr, cu, cu)
    gq, gk, gv = torch.autograd.grad(ref, (qr, kr, vr), do.float())
    lays = [compute_layout(cu, tl, cp, r, torch.device(DEV)) for r in range(cp)]
    k_loc = [k[lay.q_stream].contiguous() for lay in lays]          # what each rank holds, in its local order
    v_loc = [v[lay.q_stream].contiguous() for lay in lays]
    dk_sum = [torch.zeros(tl, nkv, d, device=DEV) for _ in range(cp)]
    dv_sum = [torch.zeros(tl, nkv, d, device=DEV) for _ in range(cp)]
    scale = d ** -0.5
    for r, lay in enumerate(lays):
        ql, dol = q[lay.q_stream].contiguous(), do[lay.q_stream].contiguous()
        o_acc = torch.zeros(tl, nq, d, device=DEV)
        lse_acc = torch.full((nq, tl), float('-inf'), device=DEV)
        for s in range(cp):
            j = (r - s) % cp
            o_s, lse_s = ac.fwd_ranges_raw(ql, k_loc[j], v_loc[j], lay.ring_lo[j], lay.ring_hi[j], scale)
            new = torch.logaddexp(lse_acc, lse_s)
            o_acc = o_acc * torch.exp(lse_acc - new).t()[..., None] + o_s.float() * torch.exp(lse_s - new).t()[..., None]
            lse_acc = new
        o = o_acc.to(torch.bfloat16)
        assert rel(o, ref[lay.q_stream]) < 2e-2
        delta = (o.float() * dol.float()).sum(-1).t().contiguous()
        dq = torch.zeros(tl, nq, d, device=DEV)
        for s in range(cp):
            j = (r - s) % cp
            dq_s, dk_s, dv_s = ac.bwd_ranges_raw(ql, k_loc[j], v_loc[j], o, dol, lse_acc, delta, lay.ring_lo[j],
                                                 lay.ring_hi[j], lay.ring_qlo[j], lay.ring_qhi[j], scale)
            dq += dq_s.float()
            dk_sum[j] += dk_s.float()
            dv_sum[j] += dv_s.float()
        assert rel(dq, gq[lay.q_stream]) < 3e-2
    for j, lay in enumerate(lays):
        assert rel(dk_sum[j], gk[lay.q_stream]) < 3e-2 and rel(dv_sum[j], gv[lay.q_stream]) < 3e-2
