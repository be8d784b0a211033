"""Fused Llama training path against the plain PyTorch evaluation of the same model."""
import pytest
import torch

from ferrotorch_b200.models import LlamaConfig, LlamaForCausalLM
from ferrotorch_b200.parallel import FSDP, AdamWConfig

pytestmark = pytest.mark.gpu


def _mk(cfg, device):
    return LlamaForCausalLM(cfg, device=device, seed=0)


def test_fused_layer_matches_reference_forward_backward():
    cfg = LlamaConfig.tiny(layers=2, hidden=256, heads=2, kv_heads=1, ffn=512, vocab=1024)
    m = _mk(cfg, "cuda")
    ref = _mk(cfg, "cpu")
    with torch.no_grad():
        for ug, uc in zip(m.units(), ref.units()):
            uc.full.copy_(ug.full.cpu())
    ids = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    labels = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    loss = m(ids, labels=labels)
    loss.backward()
    torch.cuda.synchronize()
    rl = ref(ids.cpu(), labels=labels.cpu())
    rl.backward()
    assert abs(loss.item() - rl.item()) < 3e-2 * max(1.0, abs(rl.item()))
    # gradients of the first and last layer, and the head
    for lg, lc in ((m.model.layers[0], ref.model.layers[0]), (m.model.layers[-1], ref.model.layers[-1])):
        g, r = lg.unit.grad.float().cpu(), lc.flat.grad.float()
        rel = (g - r).norm() / (r.norm() + 1e-12)
        assert rel.item() < 6e-2, rel.item()
    gh, rh = m.head_unit.grad.float().cpu(), ref.head_flat.grad.float()
    assert ((gh - rh).norm() / rh.norm()).item() < 6e-2


def test_engine_loss_decreases():
    cfg = LlamaConfig.tiny(layers=2, hidden=256, heads=2, kv_heads=1, ffn=512, vocab=512)
    m = _mk(cfg, "cuda")
    eng = FSDP(m, AdamWConfig(lr=3e-3, betas=(0.9, 0.95), weight_decay=0.0))
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    labels = torch.roll(ids, -1, 1)
    losses = []
    for _ in range(12):
        losses.append(eng.train_step(ids, labels).item())
    eng.synchronize()
    assert losses[-1] < 0.9 * losses[0], losses
