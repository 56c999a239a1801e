"""Whole-stack gradient parity: the bf16 GPU training path (tcgen05 GEMMs, fused attention, channel-major triangle
multiplication, checkpoint per block) against the same stack in fp32 on the CPU (plain PyTorch oracle), with padded
(fully masked) MSA rows and identical dropout masks.  Kernel unit tests cannot see an error that only shows when
gradients travel through several blocks; this one does.
"""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _loss(out, targets):
    return sum(((o.float() - t.float()) ** 2).mean() for o, t in zip(out, targets))


@pytest.mark.parametrize("S,N", [(32, 64), (16, 128)])
def test_stack_gradients_match_fp32_cpu(S, N, device_status, monkeypatch):
    from fastfold_b200.models.fastnn import EvoformerStack
    from fastfold_b200.models.fastnn import evoformer as evo_mod
    torch.manual_seed(3)
    c_m, c_z, c_s, n_blocks = 256, 128, 384, 3
    cpu = EvoformerStack(c_m, c_z, c_s, n_blocks, blocks_per_ckpt=1)
    g = torch.Generator().manual_seed(11)
    with torch.no_grad():
        for p in cpu.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
            p.copy_(p.to(torch.bfloat16).float())                     # both sides start from the same bf16 values
    gpu = copy.deepcopy(cpu).to("cuda", torch.bfloat16).train()
    cpu = cpu.train()
    m = torch.randn(S, N, c_m, generator=g).bfloat16()
    z = torch.randn(N, N, c_z, generator=g).bfloat16()
    msa_mask = torch.ones(S, N)
    msa_mask[[1, 5, S - 1]] = 0                                       # padded sequences: every key of their rows is masked
    pair_mask = torch.ones(N, N)
    targets = [torch.randn(S, N, c_m, generator=g), torch.randn(N, N, c_z, generator=g), torch.randn(N, c_s, generator=g)]

    draw = evo_mod.draw_block_dropout
    seeds = {"n": 0}

    def seeded_draw(n_pad, cm, cz, device, dtype, **kw):
        seeds["n"] += 1
        gen = torch.Generator().manual_seed(1000 + seeds["n"])
        masks = draw(n_pad, cm, cz, torch.device("cpu"), torch.float32, generator=gen, **kw)
        return {k: v.to(device=device, dtype=dtype) for k, v in masks.items()}

    monkeypatch.setattr(evo_mod, "draw_block_dropout", seeded_draw)
    seeds["n"] = 0
    out_c = cpu(m.float(), z.float(), msa_mask, pair_mask, None)
    loss_c = _loss(out_c, targets)
    loss_c.backward()
    seeds["n"] = 0
    out_g = gpu(m.cuda(), z.cuda(), msa_mask.cuda().bfloat16(), pair_mask.cuda().bfloat16(), None)
    loss_g = _loss(out_g, [t.cuda() for t in targets])
    loss_g.backward()
    assert abs(loss_g.item() - loss_c.item()) < 0.03 * abs(loss_c.item())
    worst = []
    gp = dict(gpu.named_parameters())
    for name, pc in cpu.named_parameters():
        gc, gg = pc.grad, gp[name].grad
        assert gg is not None and torch.isfinite(gg).all(), name
        gg = gg.float().cpu()
        ref = gc.norm().item()
        if ref < 1e-6:
            continue
        worst.append(((gg - gc).norm().item() / ref, name))
    worst.sort(reverse=True)
    assert worst[0][0] < 0.12, worst[:5]
    mean_err = sum(w for w, _ in worst) / len(worst)
    assert mean_err < 0.04, (mean_err, worst[:5])


def test_chunked_inference_paths_agree(device_status, monkeypatch):
    """No-grad forward of a 2-block stack on the GPU: un-chunked, chunked with the dense triangle multiplication, and
    chunked with the memory-bounded slab pipeline give the same result up to bf16 rounding."""
    from fastfold_b200.models.fastnn import EvoformerStack, set_chunk_size
    from fastfold_b200.models.fastnn import ops as fops
    torch.manual_seed(7)
    S, N = 32, 64
    model = EvoformerStack(256, 128, 384, 2, blocks_per_ckpt=None)
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
    model = model.to("cuda", torch.bfloat16).eval()
    m = torch.randn(S, N, 256, generator=g).bfloat16().cuda()
    z = torch.randn(N, N, 128, generator=g).bfloat16().cuda()
    mm = torch.ones(S, N)
    mm[3] = 0
    mm, pm = mm.bfloat16().cuda(), torch.ones(N, N).bfloat16().cuda()
    outs = []
    try:
        with torch.no_grad():
            outs.append(model(m, z, mm, pm, None))
            set_chunk_size(16)
            outs.append(model(m, z, mm, pm, 16))
            monkeypatch.setattr(fops, "_dense_fits", lambda *a, **k: False)
            outs.append(model(m, z, mm, pm, 16))
    finally:
        set_chunk_size(None)
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            scale = max(1.0, a.float().abs().max().item())
            assert (a.float() - b.float()).abs().max().item() < 4e-2 * scale


def test_narrow_head_attention_padded_path(device_status):
    """Heads of 8 channels (extra-MSA stack) run through the 32-channel fused attention kernel with zero-padded weights
    at inference; the result equals the composite path (taken when grad is enabled)."""
    from fastfold_b200.models.fastnn.ops import SelfAttention
    torch.manual_seed(2)
    att = SelfAttention(qkv_dim=64, c=8, n_head=8, out_dim=64, gating=True).to("cuda", torch.bfloat16).eval()
    with torch.no_grad():
        for p in att.parameters():
            p.copy_(torch.randn_like(p) * 0.25)
    x = torch.randn(1, 24, 136, 64, device="cuda").bfloat16()
    mask = (torch.rand(1, 24, 136, device="cuda") > 0.15).bfloat16()
    mask[0, 3] = 0
    bias = torch.randn(1, 8, 136, 136, device="cuda").bfloat16()
    with torch.no_grad():
        fast, _ = att(x, mask, (bias, -1))
        assert att._pad_cache is not None
    comp, _ = att.float().cpu()(x.float().cpu(), mask.float().cpu(), (bias.float().cpu(), -1))          # fp32 composite on the CPU
    comp = comp.to("cuda")
    err = (fast.float() - comp.detach().float()).abs().max().item()
    assert err < 4e-2 * max(1.0, comp.detach().float().abs().max().item()), err


def test_first_pass_uses_current_weights_after_optimizer_steps(device_status):
    """After optimiser steps that write the parameters through raw pointers (flat fused Adam), the no-grad pass of a block
    (checkpoint first pass, recycling iterations: fused kernels with derived interleaved / padded weights) must give what
    the grad-enabled pass gives with the live weights - nothing derived from an earlier step's weights may be reused."""
    from fastfold_b200.models.fastnn import EvoformerStack
    from fastfold_b200.models.fastnn.evoformer import draw_block_dropout
    from fastfold_b200.runtime import FlatAdamTrainer
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    S, N = 32, 64
    model = EvoformerStack(256, 128, 384, 1, blocks_per_ckpt=1)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.normal_(std=0.05)
    model = model.to(dev, torch.bfloat16).train()
    m = torch.randn(S, N, 256, device=dev, dtype=torch.bfloat16)
    z = torch.randn(N, N, 128, device=dev, dtype=torch.bfloat16)
    mm = torch.ones(S, N, device=dev, dtype=torch.bfloat16)
    pm = torch.ones(N, N, device=dev, dtype=torch.bfloat16)

    def loss_fn(mod, m, z, mm, pm):
        om, oz, s = mod(m, z, mm, pm, None)
        return om.float().pow(2).mean() + oz.float().pow(2).mean() + s.float().pow(2).mean()

    blk = model.blocks[0]
    drop = draw_block_dropout(N, 256, 128, dev, torch.bfloat16)
    with torch.no_grad():
        before = blk(m, z, mm, pm, _drop=drop)
    tr = FlatAdamTrainer(model, loss_fn, lr=2e-2, use_graph=False)      # large steps: stale weights would be far off
    for _ in range(3):
        tr.step(m, z, mm, pm)
    with torch.no_grad():
        first_pass = blk(m, z, mm, pm, _drop=drop)
    recomputed = blk(m.clone().requires_grad_(True), z.clone().requires_grad_(True), mm, pm, _drop=drop)
    for a, b, c in zip(first_pass, recomputed, before):
        moved = (a.float() - c.float()).abs().mean().item()
        err = (a.float() - b.detach().float()).abs().mean().item()
        assert moved > 1e-3, "the optimiser steps did not change the block's output"
        assert err < 0.1 * moved + 2e-2 * max(1.0, b.detach().float().abs().mean().item()), (err, moved)
