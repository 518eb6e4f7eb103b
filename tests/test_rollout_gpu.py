"""The rollout decode step on a GPU: grouped decode GEMM, chained launches and graph replay must agree."""
import pytest
import torch

pytestmark = pytest.mark.gpu


class _Tok:
    eos_token_id = 7
    vocab_size = 2040

    def decode(self, ids, **kw):
        return " ".join(str(int(i)) for i in ids)


def _model():
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=3, n_embd=256, vocab_size=2048, dim_att_lora=32, dim_gate_lora=64, dim_mv_lora=32,
                     eos_token_id=7)
    m = RWKV7Model(cfg)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight", "w1", "a1", "v1", "g1")):
                p.normal_(0, 0.05)
    return m.to(device="cuda", dtype=torch.bfloat16).eval()


def _rollout(model, graph: bool, chained: bool):
    from rwkvtune_b200.inference import GRPOBatchGenerator
    from rwkvtune_b200.ops import _ext

    prev = _ext.CHAINING_ALLOWED
    _ext.CHAINING_ALLOWED = chained
    try:
        gen = GRPOBatchGenerator(model, _Tok(), use_cuda_graph=graph)
        prompts = [[3, 4, 5, 6], [9, 8, 11], [100, 200, 300, 400, 500]]
        out = gen.generate(prompts, max_new_tokens=24, num_generations=4, temperature=0.0)
        torch.cuda.synchronize()
    finally:
        _ext.CHAINING_ALLOWED = prev
    return out["completion_ids"].cpu(), out["masks"].cpu()


def test_chained_graph_rollout_equals_plain_launches():
    from rwkvtune_b200.ops import gemm_native

    model = _model()
    base_ids, base_mask = _rollout(model, graph=False, chained=False)
    assert base_mask.any()
    for graph, chained in ((False, True), (True, False), (True, True)):
        ids, mask = _rollout(model, graph, chained)
        assert torch.equal(mask, base_mask), (graph, chained)
        assert torch.equal(ids, base_ids), (graph, chained)      # same kernels, same order of sums: same tokens
    assert gemm_native.check_status() == 0


def test_decode_step_logits_match_library_gemm():
    from rwkvtune_b200.inference import GRPOBatchGenerator
    from rwkvtune_b200.ops import gemm_native

    model = _model()
    gen = GRPOBatchGenerator(model, _Tok(), use_cuda_graph=False)
    tok = torch.randint(10, 2000, (16, 1), device="cuda")
    outs = []
    for dispatch in (True, False):
        prev = gemm_native.DECODE_DISPATCH
        gemm_native.DECODE_DISPATCH = dispatch
        try:
            state = gen._zero_state(16)
            with torch.no_grad():
                logits = None
                for _ in range(3):
                    logits, state = gen._forward(tok, state)
            outs.append(logits.float())
        finally:
            gemm_native.DECODE_DISPATCH = prev
    scale = outs[1].abs().max().item()
    assert (outs[0] - outs[1]).abs().max().item() <= 3e-2 * scale + 1e-2


def test_lora_decode_step_matches_ungrouped_adapter_path():
    """With LoRA adapters on all six projections the decode step runs as grouped launches (base products and x A^T
    together, B products accumulated in place); it must agree with the layer-by-layer adapter path."""
    from rwkvtune_b200 import LoraConfig
    from rwkvtune_b200.peft import get_peft_model
    from rwkvtune_b200.inference import GRPOBatchGenerator
    from rwkvtune_b200.ops import gemm_native
    from rwkvtune_b200.peft.lora.layer import LoraLinear

    model = get_peft_model(_model(), LoraConfig(r=16, lora_alpha=32))
    torch.manual_seed(3)
    n_lora = 0
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, LoraLinear):
                m.lora_B.normal_(0, 0.05)
                n_lora += 1
    assert n_lora >= 6 * 3
    model.eval()
    gen = GRPOBatchGenerator(model, _Tok(), use_cuda_graph=False)
    tok = torch.randint(10, 2000, (16, 1), device="cuda")
    outs, launches = [], []
    from rwkvtune_b200.ops import _ext
    for dispatch in (True, False):
        prev = gemm_native.DECODE_DISPATCH
        gemm_native.DECODE_DISPATCH = dispatch
        try:
            state = gen._zero_state(16)
            with torch.no_grad():
                logits = None
                for _ in range(3):
                    before = _ext.launch_count()
                    logits, state = gen._forward(tok, state)
                    launches.append(_ext.launch_count() - before)
            outs.append(logits.float())
        finally:
            gemm_native.DECODE_DISPATCH = prev
    scale = outs[1].abs().max().item()
    assert (outs[0] - outs[1]).abs().max().item() <= 3e-2 * scale + 1e-2
    assert gemm_native.check_status() == 0


@pytest.mark.parametrize("first_block", [True, False])
@pytest.mark.parametrize("pooled", [False, True])
def test_fused_decode_core_reproduces_the_three_kernel_path(first_block, pooled):
    """timemix_prep -> wkv7 -> gn_bonus_gate against the single decode-core kernel: the same values in z and in the state."""
    from rwkvtune_b200 import ops

    torch.manual_seed(7 + first_block + 2 * pooled)
    B, H = 24, 5
    C = H * 64
    dev = "cuda"
    bf = lambda s=1.0: (torch.randn(B, 1, C, device=dev) * s).to(torch.bfloat16)
    r, k, v, w_lin, a_lin, v_lin, v_first, g = bf(), bf(), bf(), bf(0.5), bf(0.5), bf(0.5), bf(), bf()
    par = lambda s=0.5: torch.nn.Parameter(torch.randn(1, 1, C, device=dev) * s)
    w0, a0, v0, k_k, k_a = par(), par(), par(), par(0.3) + 0.8, par(0.3) + 0.8
    r_k = torch.nn.Parameter(torch.randn(H, 64, device=dev) * 0.3)
    gn_w = torch.nn.Parameter(1 + 0.1 * torch.randn(C, device=dev))
    gn_b = torch.nn.Parameter(0.1 * torch.randn(C, device=dev))
    vf, vl, v0_ = (None, None, None) if first_block else (v_first, v_lin, v0)
    n_slots = 40
    pool0 = torch.randn(n_slots, H, 64, 64, device=dev) * 0.3
    slots = torch.randperm(n_slots, device=dev)[:B]
    with torch.no_grad():
        if pooled:
            pool_a, pool_b = pool0.clone(), pool0.clone()
            state_a, state_b = (pool_a, slots), (pool_b, slots)
        else:
            s0 = pool0[:B].contiguous()
            state_a, state_b = s0.clone(), s0.clone()
        w, k2, v2, a_, b_ = ops.timemix_prep(k, v, vf, w_lin, a_lin, vl, w0, a0, v0_, k_k, k_a, 64)
        z_ref, s_ref = ops.wkv7_gn(r, w, k2, v2, a_, b_, g, gn_w, gn_b, r_k, 64, state=state_a, return_state=True)
        assert ops.timemix_decode_core_ok(r, g, state_b, 64)
        z, s_new = ops.timemix_decode_core(r, k, v, vf, w_lin, a_lin, vl, g, w0, a0, v0_, k_k, k_a, r_k, gn_w, gn_b, state_b)
    torch.cuda.synchronize()

    def same(got, want, what):
        # same roundings and the same order of sums; what may differ is where the compiler contracts a multiply and an
        # add into one fused operation: a last-bit difference in an occasional element
        diff = (got.float() - want.float()).abs()
        bad = diff > 0
        assert bad.float().mean().item() < 2e-3, (what, bad.float().mean().item())
        assert (diff <= 2 ** -7 * want.float().abs() + 1e-6).all(), (what, diff.max().item())

    same(z, z_ref.to(z.dtype), "z")
    if pooled:
        same(pool_b, pool_a, "state")
        assert not torch.equal(pool_b, pool0)
    else:
        same(s_new, s_ref, "state")
        assert torch.equal(state_b, s0)      # functional: the input state is untouched


def test_fused_step_bookkeeping_equals_indexing_ops(monkeypatch):
    """Token store, length count and end-of-sequence handling in one kernel against the same statements as tensor
    indexing; many end-of-sequence ids, so that paths finish early and the batch is compacted on the way."""
    from rwkvtune_b200.inference import GRPOBatchGenerator, sampling_native

    model = _model()
    prompts = [[3, 4, 5, 6], [9, 8, 11], [100, 200, 300, 400, 500], [42]]
    outs = []
    for fused in (True, False):
        if not fused:
            monkeypatch.setattr(sampling_native, "advance_available", lambda: False)
        gen = GRPOBatchGenerator(model, _Tok(), eos_token_id=list(range(7, 160)), sync_every=2)
        out = gen.generate(prompts, max_new_tokens=40, num_generations=6, temperature=1.0, top_p=0.95, seed=1234)
        torch.cuda.synchronize()
        outs.append((out["completion_ids"].cpu(), out["masks"].cpu(), out["lengths"].cpu()))
    assert torch.equal(outs[0][2], outs[1][2])
    assert torch.equal(outs[0][1], outs[1][1]) and torch.equal(outs[0][0], outs[1][0])
    lengths = outs[0][2]
    assert (lengths < 40).any() and (lengths > 1).any()       # some paths ended on an end-of-sequence id, not all at once
