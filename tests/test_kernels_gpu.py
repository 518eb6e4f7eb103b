"""Each sm_100a kernel against the fp32 PyTorch statement of the same operator."""
import pytest
import torch

from rwkvtune_b200 import ops
from rwkvtune_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(a, b, rtol, atol, name=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    frac_bad = (err > tol).float().mean().item()
    assert frac_bad < 2e-3, f"{name}: {frac_bad:.4f} of elements off, max err {err.max().item():.4g}, ref max {b.abs().max().item():.4g}"


def _wkv_inputs(B, T, H, seed=0, dev="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    C = H * 64
    rnd = lambda s=1.0: (torch.randn(B, T, C, generator=g) * s)
    r, k, v = rnd(), rnd(), rnd()
    w = -torch.nn.functional.softplus(-(rnd(2.0) - 1.0)) - 0.5
    kk = torch.nn.functional.normalize(rnd().view(B, T, H, 64), dim=-1).view(B, T, C)
    a = torch.sigmoid(rnd())
    return [t.to(dev).to(BF) for t in (r, w, k, v, -kk, kk * a)]


@pytest.fixture
def wkv_impl():
    from rwkvtune_b200.ops import cuda_ops
    prev = cuda_ops.WKV7_IMPL

    def set_impl(name):
        cuda_ops.WKV7_IMPL = name
    yield set_impl
    cuda_ops.WKV7_IMPL = prev


def _relnorm(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("B,T,H,with_state", [(2, 64, 2, False), (1, 37, 3, True), (2, 128, 1, True), (1, 272, 2, True)])
@pytest.mark.parametrize("impl", ["simt", "tc", "tc-recompute"])
def test_wkv7_forward_backward(B, T, H, with_state, impl, wkv_impl, monkeypatch):
    from rwkvtune_b200.ops import cuda_ops
    monkeypatch.setattr(cuda_ops, "WKV7_KEEP_WORKSPACE", impl == "tc")   # "tc-recompute": backward runs its own prep pass
    impl = impl.split("-")[0]
    wkv_impl(impl)
    ins = _wkv_inputs(B, T, H)
    s0 = (torch.randn(B, H, 64, 64, device="cuda") * 0.1) if with_state else None
    ins_k = [t.clone().requires_grad_(True) for t in ins]
    ins_r = [t.float().clone().requires_grad_(True) for t in ins]
    s0_k = s0.clone().requires_grad_(True) if with_state else None
    s0_r = s0.clone().requires_grad_(True) if with_state else None
    y, sT = ops.wkv7(*ins_k, 64, state=s0_k, return_state=True)
    y_ref, sT_ref = ref.wkv7(*ins_r, 64, s0_r)
    gy = torch.randn_like(y_ref)
    gs = torch.randn_like(sT_ref) * 0.1
    (y.float() * gy).sum().add((sT * gs).sum()).backward()
    (y_ref * gy).sum().add((sT_ref * gs).sum()).backward()
    if impl == "simt":
        _close(y, y_ref, 2e-2, 2e-2, "y")
        _close(sT, sT_ref, 1e-3, 1e-3, "final state")
        for name, a, b in zip("rwkvab", ins_k, ins_r):
            _close(a.grad, b.grad, 3e-2, 3e-2 * b.grad.abs().mean().item() + 1e-3, f"d{name}")
        if with_state:
            _close(s0_k.grad, s0_r.grad, 3e-2, 3e-2 * s0_r.grad.abs().mean().item() + 1e-3, "ds0")
    else:
        # operands of the chunk products are rounded to bf16: compare in norm
        assert _relnorm(y, y_ref) < 1.5e-2
        assert _relnorm(sT, sT_ref) < 1.5e-2
        for name, a, b in zip("rwkvab", ins_k, ins_r):
            assert _relnorm(a.grad, b.grad) < 2.5e-2, (name, _relnorm(a.grad, b.grad))
        if with_state:
            assert _relnorm(s0_k.grad, s0_r.grad) < 2e-2


def test_wkv7_chunk_carry_equals_full(wkv_impl):
    wkv_impl("simt")
    ins = _wkv_inputs(1, 96, 2, seed=3)
    y_full, s_full = ops.wkv7(*ins, 64, return_state=True)
    y1, s1 = ops.wkv7(*[t[:, :40] for t in ins], 64, return_state=True)
    y2, s2 = ops.wkv7(*[t[:, 40:] for t in ins], 64, state=s1, return_state=True)
    assert torch.equal(torch.cat([y1, y2], 1), y_full)
    assert torch.allclose(s2, s_full, atol=1e-6)


def test_wkv7_tensor_core_chunk_carry(wkv_impl):
    wkv_impl("tc")
    ins = _wkv_inputs(1, 96, 2, seed=3)
    y_full, s_full = ops.wkv7(*ins, 64, return_state=True)
    y1, s1 = ops.wkv7(*[t[:, :48] for t in ins], 64, return_state=True)
    y2, s2 = ops.wkv7(*[t[:, 48:] for t in ins], 64, state=s1, return_state=True)
    # split on a chunk boundary: same products, carried state fp32 in both cases
    assert _relnorm(torch.cat([y1, y2], 1), y_full) < 1e-3
    assert _relnorm(s2, s_full) < 1e-3


@pytest.mark.parametrize("K,B,T,C,with_prev", [(6, 2, 50, 256, False), (1, 3, 17, 512, True), (6, 1, 130, 768, True)])
def test_ln_shift_mix(K, B, T, C, with_prev):
    torch.manual_seed(0)
    x = torch.randn(B, T, C, device="cuda").to(BF)
    w = (1 + 0.1 * torch.randn(C, device="cuda"))
    b = 0.1 * torch.randn(C, device="cuda")
    mix = torch.rand(K, C, device="cuda")
    prev = torch.randn(B, C, device="cuda").to(BF) if with_prev else None
    leaves_k = [t.clone().requires_grad_(True) for t in (x, w, b, mix)] + ([prev.clone().requires_grad_(True)] if with_prev else [None])
    leaves_r = [t.float().clone().requires_grad_(True) for t in (x, w, b, mix)] + ([prev.float().clone().requires_grad_(True)] if with_prev else [None])
    o, last = ops.ln_shift_mix(*leaves_k)
    o_r, last_r = ref.ln_shift_mix(*leaves_r)
    _close(o, o_r, 1e-2, 2e-2, "outs")
    _close(last, last_r, 1e-2, 2e-2, "last")
    go = torch.randn_like(o_r)
    gl = torch.randn_like(last_r)
    (o.float() * go).sum().add((last.float() * gl).sum()).backward()
    (o_r * go).sum().add((last_r * gl).sum()).backward()
    names = ["dx", "dln_w", "dln_b", "dmix", "dprev"]
    for n, a, r_ in zip(names, leaves_k, leaves_r):
        if a is None:
            continue
        scale = r_.grad.abs().mean().item()
        _close(a.grad, r_.grad, 3e-2, 3e-2 * scale + 1e-3, n)


def test_layer_norm():
    torch.manual_seed(0)
    x = torch.randn(70, 512, device="cuda").to(BF)
    w = 1 + 0.1 * torch.randn(512, device="cuda")
    b = 0.1 * torch.randn(512, device="cuda")
    lk = [t.clone().requires_grad_(True) for t in (x, w, b)]
    lr = [t.float().clone().requires_grad_(True) for t in (x, w, b)]
    y = ops.layer_norm(*lk)
    y_r = ref.layer_norm(*lr)
    _close(y, y_r, 1e-2, 1e-2, "y")
    g = torch.randn_like(y_r)
    (y.float() * g).sum().backward()
    (y_r * g).sum().backward()
    for n, a, r_ in zip(["dx", "dw", "db"], lk, lr):
        _close(a.grad, r_.grad, 3e-2, 3e-2 * r_.grad.abs().mean().item() + 1e-3, n)


@pytest.mark.parametrize("layer0", [True, False])
def test_timemix_prep(layer0):
    torch.manual_seed(1)
    B, T, C = 2, 33, 256
    big = lambda: torch.randn(B, T, C, device="cuda").to(BF)
    par = lambda s=1.0: (torch.randn(1, 1, C, device="cuda") * s)
    k, v, vf, wl, al, vl = big(), big(), big(), big(), big(), big()
    w0, a0, v0, kk, ka = par(), par(), par(), par(0.3) + 0.7, par(0.1) + 1.0
    args = [k, v, None if layer0 else vf, wl, al, None if layer0 else vl, w0, a0, None if layer0 else v0, kk, ka]
    mk = lambda f: [None if t is None else f(t).clone().requires_grad_(True) for t in args]
    ak, ar = mk(lambda t: t), mk(lambda t: t.float())
    outs = ops.timemix_prep(*ak, 64)
    outs_r = ref.timemix_prep(*ar, 64)
    gs = [torch.randn_like(o) for o in outs_r]
    for n, o, o_r in zip(["w", "k", "v", "an", "b"], outs, outs_r):
        _close(o, o_r, 1e-2, 1e-2, n)
    sum((o.float() * g).sum() for o, g in zip(outs, gs)).backward()
    sum((o * g).sum() for o, g in zip(outs_r, gs)).backward()
    names = ["dk", "dv", "dvfirst", "dwlin", "dalin", "dvlin", "dw0", "da0", "dv0", "dk_k", "dk_a"]
    for n, a, r_ in zip(names, ak, ar):
        if a is None:
            continue
        _close(a.grad, r_.grad, 3e-2, 3e-2 * r_.grad.abs().mean().item() + 1e-3, n)


def test_gn_bonus_gate():
    torch.manual_seed(2)
    B, T, C = 2, 21, 256
    big = lambda: torch.randn(B, T, C, device="cuda").to(BF)
    y, r, k, v, g = big(), big(), big(), big(), big()
    gw = 1 + 0.1 * torch.randn(C, device="cuda")
    gb = 0.1 * torch.randn(C, device="cuda")
    rk = 0.1 * torch.randn(C // 64, 64, device="cuda")
    args = [y, r, k, v, g, gw, gb, rk]
    ak = [t.clone().requires_grad_(True) for t in args]
    ar = [t.float().clone().requires_grad_(True) for t in args]
    z = ops.gn_bonus_gate(*ak, 64)
    z_r = ref.gn_bonus_gate(*ar, 64)
    _close(z, z_r, 1e-2, 2e-2, "z")
    gz = torch.randn_like(z_r)
    (z.float() * gz).sum().backward()
    (z_r * gz).sum().backward()
    for n, a, r_ in zip(["dy", "dr", "dk", "dv", "dg", "dgn_w", "dgn_b", "dr_k"], ak, ar):
        _close(a.grad, r_.grad, 3e-2, 3e-2 * r_.grad.abs().mean().item() + 1e-3, n)


def test_relu_squared():
    x = torch.randn(4, 33, 256, device="cuda").to(BF).requires_grad_(True)
    y = ops.relu_squared(x)
    xr = x.detach().float().requires_grad_(True)
    yr = ref.relu_squared(xr)
    _close(y, yr, 1e-2, 1e-3)
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    _close(x.grad, xr.grad, 2e-2, 1e-2)


def test_linear_cross_entropy_matches_reference():
    torch.manual_seed(0)
    M, C, V = 300, 128, 1024
    x = (torch.randn(M, C, device="cuda") * 0.5).to(BF)
    w = (torch.randn(V, C, device="cuda") * 0.1).to(BF)
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[:40] = -100
    xk, wk = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    loss = ops.linear_cross_entropy(xk, wk, labels, True, -100, M)
    loss_r = ref.linear_cross_entropy(xr, wr, labels, True, -100, M)
    assert abs(loss.item() - loss_r.item()) < 2e-2
    loss.backward(); loss_r.backward()
    _close(xk.grad, xr.grad, 5e-2, 5e-2 * xr.grad.abs().mean().item() + 1e-5, "dx")
    _close(wk.grad, wr.grad, 5e-2, 5e-2 * wr.grad.abs().mean().item() + 1e-5, "dw")


def test_linear_cross_entropy_over_several_slabs():
    """The head loss walks the rows in slabs of 4096 and sums the head-weight gradient over the slabs in the GEMM
    epilogue (a bf16 running sum, rounded once per slab).  3 slabs + a ragged tail against the fp32 statement, with a
    bound on what the per-slab rounding costs."""
    from rwkvtune_b200.ops import cuda_ops
    torch.manual_seed(0)
    slab = cuda_ops._LinearCrossEntropy.SLAB
    M, C, V = 3 * slab + 17, 256, 4096
    x = (torch.randn(M, C, device="cuda") * 0.5).to(BF)
    w = (torch.randn(V, C, device="cuda") * 0.05).to(BF)
    labels = torch.randint(0, V, (M,), device="cuda")
    labels[torch.rand(M, device="cuda") < 0.2] = -100
    xk, wk = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    loss = ops.linear_cross_entropy(xk, wk, labels, True, -100, M)
    loss_r = ref.linear_cross_entropy(xr, wr, labels, True, -100, M)
    assert abs(loss.item() - loss_r.item()) < 2e-2
    loss.backward(); loss_r.backward()
    assert _relnorm(xk.grad, xr.grad) < 2e-2
    # head gradient: bf16 logits-gradient operands (~0.4 % each) plus one bf16 rounding of the running sum per slab
    err = _relnorm(wk.grad, wr.grad)
    assert err < 1.2e-2, err
    # one-slab evaluation of the same problem (no running sum): the slab accumulation may not add more than 0.4 %
    cuda_ops._LinearCrossEntropy.SLAB = 1 << 20
    try:
        x1, w1 = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        ops.linear_cross_entropy(x1, w1, labels, True, -100, M).backward()
    finally:
        cuda_ops._LinearCrossEntropy.SLAB = slab
    assert abs(err - _relnorm(w1.grad, wr.grad)) < 4e-3
    assert _relnorm(wk.grad, w1.grad) < 8e-3


@pytest.mark.parametrize("temperature,with_entropy", [(1.0, True), (0.7, True), (1.3, False)])
def test_linear_logprob_entropy_matches_reference(temperature, with_entropy):
    torch.manual_seed(1)
    M, C, V = 200, 128, 1024
    x = (torch.randn(M, C, device="cuda") * 0.5).to(BF)
    w = (torch.randn(V, C, device="cuda") * 0.1).to(BF)
    targets = torch.randint(0, V, (M,), device="cuda")
    xk, wk = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    lp, ent = ops.linear_logprob_entropy(xk, wk, targets, temperature, with_entropy)
    lp_r, ent_r = ref.linear_logprob_entropy(xr, wr, targets, temperature, with_entropy)
    _close(lp, lp_r, 2e-2, 3e-2, "logp")
    g1 = torch.randn(M, device="cuda")
    total, total_r = (lp * g1).sum(), (lp_r * g1).sum()
    if with_entropy:
        _close(ent, ent_r, 2e-2, 3e-2, "entropy")
        g2 = torch.randn(M, device="cuda")
        total, total_r = total + (ent * g2).sum(), total_r + (ent_r * g2).sum()
    total.backward(); total_r.backward()
    _close(xk.grad, xr.grad, 5e-2, 5e-2 * xr.grad.abs().mean().item() + 1e-4, "dx")
    _close(wk.grad, wr.grad, 5e-2, 5e-2 * wr.grad.abs().mean().item() + 1e-4, "dw")


@pytest.mark.parametrize("with_state", [False, True])
def test_wkv7_tensor_core_long_sequence(with_state, wkv_impl):
    """Training length: 4096 steps = 256 chunk steps of carried state (bf16 chunk-boundary states in backward)."""
    wkv_impl("tc")
    B, T, H = 1, 4096, 2
    ins = _wkv_inputs(B, T, H, seed=3)
    s0 = (torch.randn(B, H, 64, 64, device="cuda") * 0.1) if with_state else None
    ins_k = [t.clone().requires_grad_(True) for t in ins]
    ins_r = [t.float().clone().requires_grad_(True) for t in ins]
    s0_k = s0.clone().requires_grad_(True) if with_state else None
    s0_r = s0.clone().requires_grad_(True) if with_state else None
    y, sT = ops.wkv7(*ins_k, 64, state=s0_k, return_state=True)
    y_ref, sT_ref = ref.wkv7(*ins_r, 64, s0_r)
    gy = torch.randn_like(y_ref)
    gs = torch.randn_like(sT_ref) * 0.1
    (y.float() * gy).sum().add((sT * gs).sum()).backward()
    (y_ref * gy).sum().add((sT_ref * gs).sum()).backward()
    assert _relnorm(y, y_ref) < 1.5e-2 and _relnorm(sT, sT_ref) < 1.5e-2
    for name, a, b in zip("rwkvab", ins_k, ins_r):
        assert _relnorm(a.grad, b.grad) < 3e-2, (name, _relnorm(a.grad, b.grad))
    # no drift along the sequence: the last quarter is as accurate as the first
    q = T // 4
    assert _relnorm(y[:, -q:], y_ref[:, -q:]) < 1.5e-2
    assert _relnorm(ins_k[0].grad[:, :q], ins_r[0].grad[:, :q]) < 3e-2


def test_wkv7_tensor_core_decay_at_its_bound(wkv_impl):
    """``w = -0.5`` everywhere is the strongest decay the model can produce (``w = -softplus(.) - 0.5``): the
    per-chunk rescaling by the inverse cumulative decay is then at its largest."""
    wkv_impl("tc")
    B, T, H = 1, 256, 2
    ins = _wkv_inputs(B, T, H, seed=5)
    ins[1] = torch.full_like(ins[1], -0.5)
    ins_k = [t.clone().requires_grad_(True) for t in ins]
    ins_r = [t.float().clone().requires_grad_(True) for t in ins]
    y, _ = ops.wkv7(*ins_k, 64)
    y_ref, _ = ref.wkv7(*ins_r, 64, None)
    gy = torch.randn_like(y_ref)
    (y.float() * gy).sum().backward()
    (y_ref * gy).sum().backward()
    assert torch.isfinite(y.float()).all()
    assert _relnorm(y, y_ref) < 1.5e-2
    for name, a, b in zip("rwkvab", ins_k, ins_r):
        assert torch.isfinite(a.grad.float()).all()
        assert _relnorm(a.grad, b.grad) < 3e-2, (name, _relnorm(a.grad, b.grad))
    # and the weakest decay the bf16 input can express (w strongly negative -> exp(-exp(w)) ~ 1)
    ins[1] = torch.full_like(ins[1], -8.0)
    ins_k = [t.clone().requires_grad_(True) for t in ins]
    ins_r = [t.float().clone().requires_grad_(True) for t in ins]
    y, _ = ops.wkv7(*ins_k, 64)
    y_ref, _ = ref.wkv7(*ins_r, 64, None)
    assert _relnorm(y, y_ref) < 1.5e-2


def test_training_step_is_bit_reproducible():
    """Same seed, same data, twice: split-K weight gradients, the sorted embedding gradient and the two-stage norm
    all use fixed orders, so parameters after two optimiser steps are bit-identical."""
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.parallel import DistContext

    def run():
        torch.manual_seed(0)
        cfg = RWKVConfig(n_layer=2, n_embd=256, vocab_size=2048, dim_att_lora=32, dim_gate_lora=64, dim_mv_lora=32)
        m = RWKV7Model(cfg)
        with torch.no_grad():
            for n, p in m.named_parameters():
                if n.endswith(("output.weight", "ffn.value.weight", "w1", "a1", "v1", "g1")):
                    p.copy_(torch.randn_like(p) * 0.05)
        eng = TrainEngine(m, EngineConfig(lr_init=1e-3, weight_decay=0.01, precision="bf16"),
                          DistContext(device=torch.device("cuda", 0)))
        g = torch.Generator().manual_seed(5)
        losses = []
        for _ in range(2):
            idx = torch.randint(0, 2048, (4, 2304), generator=g).cuda()     # 9216 rows: split-K and multi-slab paths
            losses.append(eng.train_step(idx, idx.roll(-1, 1), 1e-3).item())
        torch.cuda.synchronize()
        return losses, eng.space.params.clone()

    l1, p1 = run()
    l2, p2 = run()
    assert l1 == l2
    assert torch.equal(p1, p2)


def test_model_step_on_gpu_matches_cpu_reference():
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=256, vocab_size=1024, dim_att_lora=32, dim_gate_lora=64, dim_mv_lora=32)
    m = RWKV7Model(cfg)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight", "w1", "a1", "v1", "g1")):
                p.copy_(torch.randn_like(p) * 0.05)
    idx = torch.randint(0, 1024, (2, 48))
    labels = torch.randint(0, 1024, (2, 48))
    loss_cpu = m.loss(idx, labels)
    loss_cpu.backward()
    g_cpu = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    mg = RWKV7Model(cfg)
    mg.load_state_dict(m.state_dict())
    mg = mg.cuda().to(BF)
    loss_gpu = mg.loss(idx.cuda(), labels.cuda())
    loss_gpu.backward()
    assert abs(loss_gpu.item() - loss_cpu.item()) < 5e-2, (loss_gpu.item(), loss_cpu.item())
    bad = []
    for n, p in mg.named_parameters():
        a, b = p.grad.float().cpu(), g_cpu[n]
        if b.abs().max() <= 1e-6:
            continue
        # per-parameter relative error in norm: the bf16 model against the fp32 one (weights, activations and
        # gradients each rounded to 8 bits of mantissa through two blocks)
        rel = ((a - b).norm() / b.norm()).item()
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
        if rel > 0.08 or cos < 0.997:
            bad.append((n, round(rel, 4), round(cos, 5)))
    assert not bad, bad


def test_sampler_kernel_matches_filtered_distribution():
    from rwkvtune_b200.inference.core import TokenSampler
    from rwkvtune_b200.inference import sampling_native
    torch.manual_seed(0)
    V, n = 1000, 4096
    base = torch.randn(1, V, device="cuda") * 2.0
    logits = base.expand(n, V).contiguous()
    temp, top_p = 0.8, 0.7
    filt = TokenSampler.filter_logits(base, temp, top_p, 0, max_valid_token_id=989)
    probs = torch.softmax(filt, -1)[0]
    toks, lps = sampling_native.sample_top_p(logits, temp, top_p, 989, seed=7)
    assert toks.max() <= 989 and (probs[toks] > 0).all(), "sampled a token outside the nucleus"
    counts = torch.bincount(toks, minlength=V).float()
    kept = probs > 0
    expected = probs[kept] * n
    chi2 = ((counts[kept] - expected) ** 2 / expected.clamp(min=1e-9)).sum().item()
    dof = int(kept.sum()) - 1
    assert chi2 < dof + 6 * (2 * dof) ** 0.5 + 10, (chi2, dof)
    assert torch.allclose(lps, torch.log(probs[toks]), atol=2e-3)
    toks2, _ = sampling_native.sample_top_p(logits, temp, top_p, 989, seed=7)
    assert torch.equal(toks, toks2), "same seed must give the same draws"
    bf = sampling_native.sample_top_p(logits.to(torch.bfloat16), temp, 1.0, None, seed=3)[0]
    assert bf.min() >= 0 and bf.max() < V


@pytest.mark.parametrize("M,N,K", [(512, 512, 128), (2048, 1024, 512), (1000, 776, 200), (256, 256, 64), (4096, 2048, 2048)])
@pytest.mark.parametrize("epilogue", [0, 1, 2])
def test_gemm_on_sm_pairs_matches_reference(M, N, K, epilogue):
    """The cta_group::2 kernel (256x256 tiles over two SMs) against fp32 matmul, with ragged edges and every epilogue."""
    from rwkvtune_b200.ops import gemm_native
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda").to(BF)
    w = (torch.randn(N, K, device="cuda") * 0.2).to(BF)
    ref_out = x.float() @ w.float().t()
    if epilogue == 1:
        ref_out = torch.relu(ref_out) ** 2
        y = gemm_native.mm_nt_2cta(x, w, epilogue=1)
    elif epilogue == 2:
        res = torch.randn(M, N, device="cuda").to(BF)
        ref_out = ref_out + res.float()
        y = gemm_native.mm_nt_2cta(x, w, residual=res)
        acc = res.clone()
        y2 = gemm_native.mm_nt_2cta(x, w, out=acc)
        assert y2.data_ptr() == acc.data_ptr()
        assert (acc.float() - ref_out).abs().max().item() <= 2e-2 * ref_out.abs().max().item() + 1e-2
    else:
        y = gemm_native.mm_nt_2cta(x, w)
    torch.cuda.synchronize()
    assert gemm_native.check_status() == 0
    assert (y.float() - ref_out).abs().max().item() <= 2e-2 * ref_out.abs().max().item() + 1e-2


@pytest.mark.parametrize("M,N,K", [(512, 512, 128), (1000, 776, 200), (2048, 1024, 512), (4096, 2048, 2048)])
@pytest.mark.parametrize("layout", ["nn", "tn"])
def test_gemm_on_sm_pairs_mn_major_operands(M, N, K, layout):
    """The pair-of-SMs kernel with MN-major operands: x @ W (data gradients) and a^T @ b (weight gradients), plus the
    relu^2-derivative epilogue and store / accumulate into an existing buffer."""
    from rwkvtune_b200.ops import gemm_native
    torch.manual_seed(M * 3 + N + K)
    if layout == "nn":
        x = torch.randn(M, K, device="cuda").to(BF)
        w = (torch.randn(K, N, device="cuda") * 0.2).to(BF)
        ref_out = x.float() @ w.float()
        y = gemm_native.mm_nn_2cta(x, w)
        hidden = (torch.rand(M, N, device="cuda") * 2).to(BF)
        y5 = gemm_native.mm_nn_2cta(x, w, epilogue=5, residual=hidden)
        ref5 = ref_out * 2 * hidden.float().sqrt()
        assert (y5.float() - ref5).abs().max().item() <= 2e-2 * ref5.abs().max().item() + 1e-2
    else:
        a = torch.randn(K, M, device="cuda").to(BF)
        b = (torch.randn(K, N, device="cuda") * 0.2).to(BF)
        ref_out = a.float().t() @ b.float()
        y = gemm_native.mm_tn_2cta(a, b)
        buf = torch.full((M, N), 7.0, device="cuda").to(BF)
        gemm_native.mm_tn_2cta(a, b, out=buf, accumulate=False)
        assert (buf.float() - ref_out).abs().max().item() <= 2e-2 * ref_out.abs().max().item() + 1e-2
        gemm_native.mm_tn_2cta(a, b, out=buf)
        assert (buf.float() - 2 * ref_out).abs().max().item() <= 4e-2 * ref_out.abs().max().item() + 2e-2
    torch.cuda.synchronize()
    assert gemm_native.check_status() == 0
    assert (y.float() - ref_out).abs().max().item() <= 2e-2 * ref_out.abs().max().item() + 1e-2


def _chi_square_ok(toks, probs, n):
    V = probs.numel()
    counts = torch.bincount(toks, minlength=V).float()
    kept = probs > 0
    assert (probs[toks] > 0).all(), "sampled a token outside the allowed set"
    expected = probs[kept] * n
    chi2 = ((counts[kept] - expected) ** 2 / expected.clamp(min=1e-9)).sum().item()
    dof = max(int(kept.sum()) - 1, 1)
    assert chi2 < dof + 6 * (2 * dof) ** 0.5 + 10, (chi2, dof)


@pytest.mark.parametrize("top_k,top_p", [(50, 1.0), (20, 0.8), (0, 0.6)])
def test_sampler_kernel_topk_bias_and_penalty_match_the_filter(top_k, top_p):
    """The fused sampler against the statement-by-statement rule (penalty from the seen bitmap, ban, temperature,
    bias, top-k, top-p) on the distribution of many draws from one row."""
    from rwkvtune_b200.inference.core import TokenSampler, apply_repetition_penalty
    from rwkvtune_b200.inference import sampling_native
    torch.manual_seed(1)
    V, n = 1200, 4096
    base = torch.randn(1, V, device="cuda") * 2.0
    logits = base.expand(n, V).contiguous()
    bias = {3: 4.0, 17: -150.0, 900: 2.5, 5000: 1.0}
    seen1 = torch.zeros(1, V, dtype=torch.bool, device="cuda")
    seen1[0, torch.randperm(V, device="cuda")[:200]] = True
    seen = seen1.expand(n, V).contiguous()
    temp, pen = 0.9, 1.3
    ref_logits = apply_repetition_penalty(base.clone(), seen1, pen)
    filt = TokenSampler.filter_logits(ref_logits, temp, top_p, top_k, bias, max_valid_token_id=1100)
    probs = torch.softmax(filt, -1)[0]
    toks, lps = sampling_native.sample_tokens(logits, temp, top_p, top_k, bias, 1100, seen=seen,
                                              repetition_penalty=pen, update_seen=True, seed=11)
    _chi_square_ok(toks, probs, n)
    assert torch.allclose(lps, torch.log(probs[toks]), atol=3e-3)
    if top_k:
        assert int((probs > 0).sum()) <= top_k
    # the drawn token was marked in each row's bitmap, nothing else changed
    after = seen.clone()
    expect = seen1.expand(n, V).clone()
    expect[torch.arange(n, device="cuda"), toks] = True
    assert torch.equal(after, expect)
    # rows indexed through seen_rows: batch row i uses bitmap row perm[i]
    perm = torch.randperm(n, device="cuda")
    seen2 = torch.zeros(n, V, dtype=torch.bool, device="cuda")
    t2, _ = sampling_native.sample_tokens(logits, temp, top_p, top_k, None, None, seen=seen2, seen_rows=perm,
                                          repetition_penalty=pen, update_seen=True, seed=5)
    assert torch.equal(seen2[perm, t2], torch.ones(n, dtype=torch.bool, device="cuda")) and int(seen2.sum()) == n


def test_sampler_kernel_greedy_and_sample_batch_routing():
    from rwkvtune_b200.inference.core import TokenSampler
    from rwkvtune_b200.inference import sampling_native
    torch.manual_seed(2)
    n, V = 64, 65536
    logits = (torch.randn(n, V, device="cuda") * 3).to(BF)
    bias = {7: 50.0}
    tok, lp = sampling_native.sample_tokens(logits, 0.0, 0.5, 10, bias, 65529, seed=1)
    ref = logits.float().clone()
    ref[:, 65530:] = float("-inf")
    ref[:, 7] += 50.0
    assert torch.equal(tok, ref.argmax(-1))
    assert torch.allclose(lp, torch.log_softmax(ref, -1).gather(1, tok[:, None]).squeeze(1), atol=2e-3)
    # TokenSampler.sample_batch goes through the kernel for every combination without a logits_processor
    prev = TokenSampler._max_valid_token_id
    TokenSampler.set_max_valid_token_id(65529)
    try:
        t1, l1 = TokenSampler.sample_batch(logits, 0.8, 0.9, 40, bias, seed=9)
        t2, l2 = sampling_native.sample_tokens(logits, 0.8, 0.9, 40, bias, 65529, seed=9)
        assert torch.equal(t1, t2) and torch.equal(l1, l2)
        filt = TokenSampler.filter_logits(logits, 0.8, 0.9, 40, bias)
        assert torch.isfinite(filt.gather(1, t1[:, None])).all()
    finally:
        TokenSampler.set_max_valid_token_id(prev)


@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (200, 320, 96), (1024, 2048, 2048), (384, 64, 32)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_tcgen05_gemm_layouts(M, N, K, layout):
    from rwkvtune_b200.ops import gemm_native
    if not gemm_native.available():
        pytest.fail("native GEMM missing from the library")
    torch.manual_seed(M + N + K)
    if layout == "nt":
        a = torch.randn(M, K, device="cuda").to(BF); b = torch.randn(N, K, device="cuda").to(BF)
        ref_out = a.float() @ b.float().t()
        assert gemm_native.native_ok(a, b, "nt")
        out = gemm_native.mm_nt(a, b)
    elif layout == "nn":
        a = torch.randn(M, K, device="cuda").to(BF); b = torch.randn(K, N, device="cuda").to(BF)
        ref_out = a.float() @ b.float()
        out = gemm_native.mm_nn(a, b)
    else:
        a = torch.randn(K, M, device="cuda").to(BF); b = torch.randn(K, N, device="cuda").to(BF)
        ref_out = a.float().t() @ b.float()
        out = gemm_native.mm_tn(a, b)
    torch.cuda.synchronize()
    assert gemm_native.check_status() == 0, "a device-side wait in the GEMM kernel timed out"
    err = (out.float() - ref_out).abs().max().item()
    assert err <= 2e-2 * ref_out.abs().max().item() + 1e-2, (layout, err, ref_out.abs().max().item())


def test_tcgen05_gemm_relu_sq_epilogue():
    from rwkvtune_b200.ops import gemm_native
    torch.manual_seed(0)
    a = torch.randn(512, 256, device="cuda").to(BF); b = torch.randn(768, 256, device="cuda").to(BF)
    out = gemm_native.mm_nt(a, b, epilogue=1)
    ref_out = torch.relu(a.float() @ b.float().t()) ** 2
    assert gemm_native.check_status() == 0
    assert (out.float() - ref_out).abs().max().item() <= 2e-2 * ref_out.abs().max().item() + 1e-2


@pytest.mark.parametrize("M,N,K,W,rank", [(512, 512, 512, 4, 1), (1024, 2560, 2560, 8, 5), (384, 320, 256, 2, 0)])
def test_ag_fused_gemm_emulated_panels(M, N, K, W, rank):
    """K-panels of the weight held in separate buffers (as if on W ranks); the fused kernel must gather them into
    the staging matrix and produce x @ W^T.  Called repeatedly to check the running arrival counters."""
    from rwkvtune_b200.ops import gemm_native
    torch.manual_seed(K)
    x = torch.randn(M, K, device="cuda").to(BF)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(BF)
    Kp = K // W
    shards = [w[:, p * Kp:(p + 1) * Kp].contiguous() for p in range(W)]
    gw = gemm_native.GatheredWeight([s.data_ptr() for s in shards], rank, W, N, K, x.device, n_copy=8)
    ref_out = x.float() @ w.float().t()
    for _ in range(2):
        gw.staged.zero_()
        y = gemm_native.ag_mm_nt(x, gw)
        torch.cuda.synchronize()
        assert gemm_native.check_status() == 0
        assert torch.equal(gw.staged, w)
        assert (y.float() - ref_out).abs().max().item() <= 2e-2 * ref_out.abs().max().item() + 1e-2
    # a different row count on the same buffers: another grid size, so another number of arrivals per counter
    gw.staged.zero_()
    y = gemm_native.ag_mm_nt(x[:256].contiguous(), gw)
    torch.cuda.synchronize()
    assert gemm_native.check_status() == 0 and torch.equal(gw.staged, w)
    assert (y.float() - ref_out[:256]).abs().max().item() <= 2e-2 * ref_out.abs().max().item() + 1e-2
    # an appended local operand pair (the LoRA term of a sharded weight): y = x W^T + u v^T in the same launch
    u = (torch.randn(M, 64, device="cuda") * 0.5).to(BF)
    v = (torch.randn(N, 64, device="cuda") * 0.1).to(BF)
    gw.staged.zero_()
    y = gemm_native.ag_mm_nt(x, gw, u, v)
    torch.cuda.synchronize()
    ref2 = ref_out + u.float() @ v.float().t()
    assert gemm_native.check_status() == 0 and torch.equal(gw.staged, w)
    assert (y.float() - ref2).abs().max().item() <= 2e-2 * ref2.abs().max().item() + 1e-2
    # ... with relu^2, and with a residual, in the same launch's epilogue
    y = gemm_native.ag_mm_nt(x, gw, u, v, epilogue=1)
    res = torch.randn(M, N, device="cuda").to(BF)
    y2 = gemm_native.ag_mm_nt(x, gw, u, v, residual=res)
    torch.cuda.synchronize()
    assert gemm_native.check_status() == 0
    want = torch.relu(ref2) ** 2
    assert (y.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-2
    want = ref2 + res.float()
    assert (y2.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-2


@pytest.mark.parametrize("B,T,H,with_state", [(2, 64, 2, False), (1, 37, 3, True), (2, 256, 1, True)])
def test_wkv7_tensor_core_forward(B, T, H, with_state):
    from rwkvtune_b200.ops import cuda_ops
    ins = _wkv_inputs(B, T, H, seed=5)
    s0 = (torch.randn(B, H, 64, 64, device="cuda") * 0.1) if with_state else None
    y, sT, cs = cuda_ops.wkv7_tc_forward(*ins, state=s0, return_state=True, save_chunk_states=True)
    y_ref, sT_ref = ref.wkv7(*[t.float() for t in ins], 64, s0)
    rel = ((y.float() - y_ref).norm() / y_ref.norm()).item()
    assert rel < 1.5e-2, rel
    rel_s = ((sT - sT_ref).norm() / sT_ref.norm()).item()
    assert rel_s < 1.5e-2, rel_s
    if with_state:
        assert torch.allclose(cs[:, :, 0].float(), s0, atol=2e-2, rtol=2e-2)


def test_gather_rows_and_embedding():
    torch.manual_seed(0)
    V, C, M = 500, 256, 3000
    w = torch.randn(V, C, device="cuda").to(BF)
    idx = torch.randint(0, V, (4, M // 4), device="cuda")
    idx[0, :50] = 7    # a heavily repeated token
    wk = w.clone().requires_grad_(True)
    wr = w.float().clone().requires_grad_(True)
    y = ops.embedding(idx, wk)
    yr = torch.nn.functional.embedding(idx, wr)
    assert torch.equal(y.float(), yr)
    g = torch.randn_like(yr).to(BF)
    (y.float() * g.float()).sum().backward()
    (yr * g.float()).sum().backward()
    _close(wk.grad, wr.grad, 1e-2, 1e-2, "dW")
    # state fan-out / compaction on fp32 [n, H, 64, 64] rows
    st = torch.randn(6, 2, 64, 64, device="cuda")
    sel = torch.tensor([0, 0, 0, 5, 2, 2], device="cuda")
    assert torch.equal(ops.gather_rows(st, sel), st.index_select(0, sel))


@pytest.mark.parametrize("M", [1, 7, 64, 100, 128])
def test_decode_grouped_gemm(M):
    """Cluster split-K decode GEMM: both weight layouts, ragged N and K, every epilogue, residual add, every split."""
    from rwkvtune_b200.ops import gemm_native
    torch.manual_seed(M)
    # (N, K, weight stored [K, N], epilogue, residual)
    probs = [(256, 512, False, None, False), (1024, 512, False, "relu_sq", True), (72, 2048, True, "tanh", False),
             (512, 96, True, None, True), (200, 264, False, "sigmoid", False), (2048, 64, True, None, False)]
    xs = [(torch.randn(M, K, device="cuda") * 0.5).to(BF) for _, K, *_ in probs]
    ws = [((torch.randn(K, N, device="cuda") if kn else torch.randn(N, K, device="cuda")) * 0.05).to(BF)
          for N, K, kn, _, _ in probs]
    res = [torch.randn(M, N, device="cuda").to(BF) if r else None for N, _, _, _, r in probs]
    kn = [p[2] for p in probs]
    epis = [p[3] for p in probs]
    assert all(gemm_native.decode_ok(x, w, t) for x, w, t in zip(xs, ws, kn))
    act = {None: lambda t: t, "relu_sq": lambda t: torch.relu(t) ** 2, "tanh": torch.tanh, "sigmoid": torch.sigmoid}
    refs = []
    for x, w, t, e, r in zip(xs, ws, kn, epis, res):
        y = act[e](x.float() @ (w.float() if t else w.float().t()))
        refs.append(y + r.float() if r is not None else y)
    first = None
    for split in (0, 1, 2, 4, 8):
        ys = gemm_native.decode_group(xs, ws, epis=epis, kn=kn, residuals=res, split=split)
        for y, ref_y in zip(ys, refs):
            assert (y.float() - ref_y).abs().max().item() <= 1e-2 * ref_y.abs().max().item() + 1e-2, split
        if split == 0:
            first = ys
    again = gemm_native.decode_group(xs, ws, epis=epis, kn=kn, residuals=res)
    for a, b in zip(first, again):
        assert torch.equal(a, b)          # fixed summation order: bit-reproducible
    assert gemm_native.check_status() == 0
    with torch.no_grad():       # the front-end routes decode-sized groups here
        outs = ops.linear_group([xs[0], xs[1]], [ws[0], ws[1]])
    assert (outs[0].float() - xs[0].float() @ ws[0].float().t()).abs().max().item() <= 2e-2


def test_decode_gemm_residual_in_place():
    from rwkvtune_b200.ops import gemm_native
    torch.manual_seed(5)
    x = (torch.randn(64, 2048, device="cuda") * 0.5).to(BF)
    w = (torch.randn(2048, 2048, device="cuda") * 0.03).to(BF)
    r = torch.randn(64, 2048, device="cuda").to(BF)
    (y,) = gemm_native.decode_group([x], [w], residuals=[r])
    ref_y = x.float() @ w.float().t() + r.float()
    assert (y.float() - ref_y).abs().max().item() <= 1e-2 * ref_y.abs().max().item() + 1e-2


@pytest.mark.parametrize("layout", ["nt", "nn"])
@pytest.mark.parametrize("K2", [64, 16, 136])
def test_gemm_second_operand_pair_along_k(layout, K2):
    """x W^T + x2 W2^T (and the NN form) as one launch: the second pair's K blocks follow the first pair's in the ring."""
    from rwkvtune_b200.ops import gemm, gemm_native
    torch.manual_seed(K2)
    M, K, N = 4096, 328, 3200          # ragged last K block of the first pair; enough 256x256 tiles for the pair kernel
    x = (torch.randn(M, K, device="cuda") * 0.5).to(BF)
    x2 = (torch.randn(M, K2, device="cuda") * 0.5).to(BF)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(BF)
    w2 = (torch.randn(N, K2, device="cuda") * 0.1).to(BF)
    ref_y = x.float() @ w.float().t() + x2.float() @ w2.float().t()
    if layout == "nt":
        assert gemm_native.dual_ok(x, w, x2, w2, "nt")
        y = gemm.mm_nt_plus(x, w, x2, w2)
    else:
        wt, w2t = w.t().contiguous(), w2.t().contiguous()
        assert gemm_native.dual_ok(x, wt, x2, w2t, "nn")
        y = gemm.mm_nn_plus(x, wt, x2, w2t)
    assert (y.float() - ref_y).abs().max().item() <= 1e-2 * ref_y.abs().max().item() + 1e-2
    assert gemm_native.check_status() == 0


@pytest.mark.parametrize("mode", ["plain", "residual", "relu_sq"])
def test_lora_linear_single_launch_forward_and_dgrad(mode):
    """LoRA linear at a training shape: y and dx each come from one GEMM launch with the rank-r term appended to the
    contraction, the residual sum or relu^2 in that launch's epilogue; values and all gradients against the fp32
    statement of the same layer."""
    from rwkvtune_b200.ops import _ext
    from rwkvtune_b200.peft.lora.layer import LoraLinear
    torch.manual_seed(11)
    M, Cin, Cout, r = 4096, 2048, 3072, 64
    base = torch.nn.Linear(Cin, Cout, bias=False, device="cuda", dtype=BF)
    base.weight.requires_grad_(False)
    layer = LoraLinear(base, r=r, lora_alpha=2 * r)
    with torch.no_grad():
        layer.lora_B.normal_(0, 0.02)
    x = (torch.randn(M, Cin, device="cuda") * 0.5).to(BF).requires_grad_(True)
    res = torch.randn(M, Cout, device="cuda").to(BF).requires_grad_(True) if mode == "residual" else None
    dy = (torch.randn(M, Cout, device="cuda") * 0.1).to(BF)
    before = _ext.launch_count()
    y = layer(x, residual=res, act="relu_sq" if mode == "relu_sq" else None)
    fwd_launches = _ext.launch_count() - before
    y.backward(dy)
    assert fwd_launches == 2            # x A^T, then the base product with the adapter term as its last K block
    xf, W, A, B = x.detach().float(), base.weight.float(), layer.lora_A.float(), layer.lora_B.float()
    s = layer.scaling
    pre = xf @ W.t() + s * (xf @ A.t()) @ B.t()
    if mode == "relu_sq":
        ref_y = torch.relu(pre) ** 2
        dpre = dy.float() * 2 * torch.relu(pre)
    else:
        ref_y = pre + (res.detach().float() if res is not None else 0)
        dpre = dy.float()
    ref_dx = dpre @ W + s * (dpre @ B) @ A
    ref_da = s * (dpre @ B).t() @ xf
    ref_db = s * dpre.t() @ (xf @ A.t())
    for got, want in ((y, ref_y), (x.grad, ref_dx), (layer.lora_A.grad, ref_da), (layer.lora_B.grad, ref_db)):
        assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 1e-2
    if res is not None:
        assert torch.equal(res.grad, dy)


@pytest.mark.parametrize("layout", ["nt", "nn"])
def test_gemm_accumulate_epilogue(layout):
    from rwkvtune_b200.ops import gemm
    torch.manual_seed(3)
    M, K, N = 1000, 64, 520            # ragged M and N tiles, LoRA-like short contraction
    x = (torch.randn(M, K, device="cuda") * 0.5).to(BF)
    w = (torch.randn(N, K, device="cuda") * 0.2).to(BF)
    y0 = torch.randn(M, N, device="cuda").to(BF)
    y = y0.clone()
    if layout == "nt":
        out = gemm.addmm_nt_(y, x, w)
    else:
        out = gemm.addmm_nn_(y, x, w.t().contiguous())
    assert out.data_ptr() == y.data_ptr()
    ref_y = y0.float() + x.float() @ w.float().t()
    assert (y.float() - ref_y).abs().max().item() <= 2e-2 * ref_y.abs().max().item() + 1e-2


@pytest.mark.parametrize("M,N,Kc", [(2048, 96, 16384), (96, 2048, 16384), (320, 264, 9000)])
def test_gemm_split_k_weight_gradient(M, N, Kc):
    """Few output tiles, long contraction (weight gradients of the low-rank maps): split-K on the tcgen05 kernel."""
    from rwkvtune_b200.ops import gemm, gemm_native
    torch.manual_seed(5)
    a = (torch.randn(Kc, M, device="cuda") * 0.5).to(BF)
    b = (torch.randn(Kc, N, device="cuda") * 0.5).to(BF)
    splits = gemm_native.splitk_plan(a, b)
    assert splits >= 2
    out = gemm.mm_tn(a, b)
    ref_y = a.float().t() @ b.float()
    assert out.shape == (M, N) and out.dtype == BF
    assert (out.float() - ref_y).abs().max().item() <= 1e-2 * ref_y.abs().max().item()
    assert gemm_native.check_status() == 0
    # a slice count that does not divide the K blocks evenly
    out2 = gemm_native.mm_tn_splitk(a, b, 7)
    assert (out2.float() - ref_y).abs().max().item() <= 1e-2 * ref_y.abs().max().item()


@pytest.mark.parametrize("act", ["tanh", "sigmoid"])
def test_gemm_activation_epilogue(act):
    torch.manual_seed(4)
    M, K, N = 700, 256, 96
    x = (torch.randn(M, K, device="cuda") * 0.5).to(BF)
    w = (torch.randn(K, N, device="cuda") * 0.2).to(BF)
    xk, wk = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    y = ops.matmul_act(xk, wk, act)
    pre = xr @ wr
    yr = torch.tanh(pre) if act == "tanh" else torch.sigmoid(pre)
    _close(y, yr, 1e-2, 1e-2, act)
    g = torch.randn_like(yr)
    (y.float() * g).sum().backward()
    (yr * g).sum().backward()
    _close(xk.grad, xr.grad, 3e-2, 3e-2 * xr.grad.abs().mean().item() + 1e-3, "dx")
    _close(wk.grad, wr.grad, 3e-2, 3e-2 * wr.grad.abs().mean().item() + 1e-2, "dw")


@pytest.mark.parametrize("T", [1, 5])
def test_wkv7_pool_step_updates_slots_in_place(T):
    B, H = 3, 2
    ins = _wkv_inputs(B, T, H, seed=9)
    pool = torch.randn(7, H, 64, 64, device="cuda") * 0.1
    slots = torch.tensor([5, 0, 3], device="cuda")
    before = pool.clone()
    y = ops.wkv7_pool_step(*ins, pool, slots)
    y_ref, s_ref = ref.wkv7(*[t.float() for t in ins], 64, before.index_select(0, slots))
    _close(y, y_ref, 2e-2, 2e-2, "y")
    assert torch.allclose(pool.index_select(0, slots), s_ref, atol=1e-3, rtol=1e-3)
    untouched = torch.tensor([1, 2, 4, 6], device="cuda")
    assert torch.equal(pool.index_select(0, untouched), before.index_select(0, untouched))


def test_scheduler_pool_step_matches_gathered_states():
    """The scheduler's in-place pool step gives the logits and states of the gather / compute / scatter formulation."""
    from rwkvtune_b200.inference import SchedulerCore
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    class Tok:
        eos_token_id = 7
        vocab_size = 250
        idx2token = {i: bytes([65 + i % 26]) for i in range(1, 250)}

        def decode(self, ids, **kw):
            return "".join(chr(65 + int(i) % 26) for i in ids)

    torch.manual_seed(0)
    m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=128, vocab_size=256, eos_token_id=7, dim_att_lora=16, dim_gate_lora=16,
                              dim_mv_lora=16))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight", "w1", "a1", "v1", "g1")):
                p.normal_(0, 0.05)
    m = m.cuda().to(BF).eval()
    sched = SchedulerCore(m, Tok(), max_batch_size=4, max_batch_tokens=16, prefill_chunk_size=4)
    for k, pool in sched.state_pool.items():
        pool.copy_(torch.randn_like(pool.float()).to(pool.dtype) * 0.1)
    before = {k: v.clone() for k, v in sched.state_pool.items()}
    slots = [2, 0, 3]
    idx = torch.tensor(slots, device="cuda")
    ids = torch.randint(1, 250, (3, 3), device="cuda")
    logits = sched._model_forward_with_state(ids, slots)
    with torch.no_grad():
        x, a, s, f = m.forward_states(ids, list(before["att_x_prev"].index_select(1, idx).unbind(0)),
                                      list(before["att_kv"].index_select(1, idx).unbind(0)),
                                      list(before["ffn_x_prev"].index_select(1, idx).unbind(0)))
        ref_logits = m.head(x[:, -1, :]).float()
    assert torch.allclose(logits, ref_logits, atol=2e-2, rtol=2e-2)
    assert torch.allclose(sched.state_pool["att_kv"].index_select(1, idx), torch.stack(s).float(), atol=1e-4, rtol=1e-4)
    assert torch.equal(sched.state_pool["att_kv"][:, 1], before["att_kv"][:, 1])      # slot 1 was not scheduled


def test_channel_mix_ffn_fused_node():
    torch.manual_seed(5)
    M, C = 640, 256
    xk = (torch.randn(2, M // 2, C, device="cuda") * 0.5).to(BF)
    res = torch.randn(2, M // 2, C, device="cuda").to(BF)
    wk = (torch.randn(4 * C, C, device="cuda") * 0.05).to(BF)
    wv = (torch.randn(C, 4 * C, device="cuda") * 0.05).to(BF)
    leaves_k = [t.clone().requires_grad_(True) for t in (xk, wk, wv, res)]
    leaves_r = [t.float().clone().requires_grad_(True) for t in (xk, wk, wv, res)]
    out = ops.channel_mix_ffn(*leaves_k)
    out_r = leaves_r[3] + torch.relu(leaves_r[0] @ leaves_r[1].t()) ** 2 @ leaves_r[2].t()
    _close(out, out_r, 2e-2, 2e-2, "out")
    g = torch.randn_like(out_r)
    (out.float() * g).sum().backward()
    (out_r * g).sum().backward()
    for name, a, b in zip(["dxk", "dwk", "dwv", "dres"], leaves_k, leaves_r):
        _close(a.grad, b.grad, 4e-2, 4e-2 * b.grad.abs().mean().item() + 1e-3, name)


@pytest.mark.parametrize("with_state", [False, True])
def test_wkv7_gn_fused_node_matches_reference(with_state):
    B, T, H = 2, 80, 2
    C = H * 64
    ins = _wkv_inputs(B, T, H, seed=11)
    torch.manual_seed(12)
    g = torch.sigmoid(torch.randn(B, T, C, device="cuda")).to(BF)
    gn_w = 1 + 0.1 * torch.randn(C, device="cuda")
    gn_b = 0.1 * torch.randn(C, device="cuda")
    r_k = 0.1 * torch.randn(H, 64, device="cuda")
    s0 = (torch.randn(B, H, 64, 64, device="cuda") * 0.1) if with_state else None
    lk = [t.clone().requires_grad_(True) for t in (*ins, g, gn_w, gn_b, r_k)]
    lr = [t.float().clone().requires_grad_(True) for t in (*ins, g, gn_w, gn_b, r_k)]
    sk = s0.clone().requires_grad_(True) if with_state else None
    sr = s0.clone().requires_grad_(True) if with_state else None
    z, sT = ops.wkv7_gn(*lk, 64, state=sk, return_state=True)
    y_r, sT_r = ref.wkv7(*lr[:6], 64, sr)
    z_r = ref.gn_bonus_gate(y_r, lr[0], lr[2], lr[3], lr[6], lr[7], lr[8], lr[9], 64)
    assert _relnorm(z, z_r) < 2e-2 and _relnorm(sT, sT_r) < 1.5e-2
    gz = torch.randn_like(z_r)
    gs = torch.randn_like(sT_r) * 0.1
    (z.float() * gz).sum().add((sT * gs).sum()).backward()
    (z_r * gz).sum().add((sT_r * gs).sum()).backward()
    for name, a_, b_ in zip(["dr", "dw", "dk", "dv", "da", "db", "dg", "dgn_w", "dgn_b", "dr_k"], lk, lr):
        assert _relnorm(a_.grad, b_.grad) < 3e-2, (name, _relnorm(a_.grad, b_.grad))
    if with_state:
        assert _relnorm(sk.grad, sr.grad) < 2e-2
