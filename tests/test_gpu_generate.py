"""Incremental decoding of the hybrid LM over the DSQG rings against re-running the whole prefix
(which is what the reference's generate() does, train/train_2048_condU.py:463-487)."""
import pytest
import torch

from dwarf_b200.model import CondMLM
from tests.gpu_util import rel_inf

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def small_model(offsets, seq_len=160, attention="condU"):
    torch.manual_seed(7)
    m = CondMLM(vocab=211, dim=64, heads=2, layers=3, ffn=128, seq_len=seq_len,
                full_attention_layer=1, offsets=offsets, attention=attention).to(DEV).eval()
    with torch.no_grad():          # the zero/one initial values would hide these terms
        for blk in m.blocks:
            if hasattr(blk.attn, "scale_embed"):
                blk.attn.scale_embed.normal_(0.0, 0.05)
                blk.attn.if_gain.uniform_(0.8, 1.2)
        for p in m.parameters():   # N(0, 0.02) weights give nearly constant logits: widen them
            if p.dim() == 2:
                p.mul_(8.0)
    return m


@pytest.mark.parametrize("offsets,prompt", [((0, 1, 2, 3, 4, 8, 16, 48), 70),     # ring of 49 slots wraps
                                            ((0, 1, 2, 3, 5, 64, 150), 9)])       # ring longer than the text
@pytest.mark.parametrize("attention", ["condU", "condM"])
def test_decode_token_logits_equal_full_recompute(offsets, prompt, attention):
    m = small_model(offsets, attention=attention)
    S, new = 3, 24
    ids = torch.randint(0, 211, (S, prompt + new), device=DEV, generator=torch.Generator(DEV).manual_seed(1))
    full = m(ids).float()                                   # logits of every position, one pass
    logits, state = m.prefill(ids[:, :prompt], max_len=prompt + new)
    assert rel_inf(logits.float().cpu(), full[:, prompt - 1].cpu()) < 2e-2
    for t in range(prompt, prompt + new):
        logits = m.decode_token(ids[:, t], state)
        assert rel_inf(logits.float().cpu(), full[:, t].cpu()) < 2e-2, f"position {t}"
    assert state["t"] == prompt + new


def test_generate_is_deterministic_and_extends_the_prompt():
    m = small_model((0, 1, 2, 3, 4, 8, 16, 48))
    ids = torch.randint(0, 211, (2, 50), device=DEV, generator=torch.Generator(DEV).manual_seed(2))
    a = m.generate(ids, 12)
    b = m.generate(ids, 12)
    assert a.shape == (2, 62) and torch.equal(a[:, :50], ids) and torch.equal(a, b)
    # the first new token is the argmax of the full model's last-position logits
    assert torch.equal(a[:, 50], m(ids)[:, -1].argmax(-1))
    with pytest.raises(ValueError):
        m.generate(torch.zeros(1, 150, dtype=torch.long, device=DEV), 20)      # beyond seq_len 160
