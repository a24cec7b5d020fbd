"""The attention drop-in (model.py:59-152) against the reference's own Attention class from
oracle/_ref: same parameters through the strict state_dict, bf16 on the GPU against the
reference in fp32 on the CPU on bf16-rounded values."""
import pytest
import torch

from gemmallm_b200 import Attention
from oracle import make_ref

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not make_ref.available(), reason="oracle/_ref/model.py absent")]
DT = torch.bfloat16


def build_pair(hidden, hd, qh, kvh, ctx, seed, dev):
    ref = make_ref.load()
    torch.manual_seed(seed)
    emb = ref.ROPEEmbedding(ctx, head_dim=hd)
    ra = ref.Attention(hidden, hd, qh, kvh, emb).eval()
    with torch.no_grad():
        for n, p in ra.named_parameters():
            if "pos_emb" in n:
                continue
            p.copy_((torch.randn_like(p) * (0.05 if p.dim() > 1 else 0.1)).to(DT).float())
    new = Attention(hidden, hd, qh, kvh, ref.ROPEEmbedding(ctx, head_dim=hd)).eval()
    new.load_state_dict(ra.state_dict(), strict=True)
    assert list(new.state_dict()) == list(ra.state_dict())
    return ra, new.to(device=dev, dtype=DT)


@pytest.mark.parametrize("B,S,hidden,qh,kvh,masked,ft", [
    (3, 64, 1024, 16, 1, True, False), (2, 64, 256, 4, 4, False, False), (5, 37, 256, 4, 2, True, True),
    (1, 128, 128, 2, 1, True, False), (2, 1, 128, 2, 2, False, False), (64, 64, 1024, 16, 1, True, False)])
def test_attention_matches_the_reference_class(cuda_device, B, S, hidden, qh, kvh, masked, ft):
    hd = 64
    ra, new = build_pair(hidden, hd, qh, kvh, 128, B + S, cuda_device)
    x = (torch.randn(B, S, hidden, generator=torch.Generator().manual_seed(S))).to(DT).float()
    mask = torch.triu(torch.full((S, S), float("-inf")), diagonal=1) if masked else None
    with torch.no_grad():
        want = ra(x.clone(), attention_mask=mask, fine_tuning=ft)
        got = new(x.to(DT).to(cuda_device), attention_mask=None if mask is None else mask.to(cuda_device),
                  fine_tuning=ft)
        again = new(x.to(DT).to(cuda_device), attention_mask=None if mask is None else mask.to(cuda_device),
                    fine_tuning=ft)
    torch.cuda.synchronize()
    assert torch.equal(got, again)
    err = (got.float().cpu() - want).abs().max()
    # bf16 path (QKV, probabilities and the output Linear round to bf16): relative 2e-2
    assert err <= 2e-2 * want.abs().max(), f"max-abs {err} vs scale {want.abs().max()}"
    assert (got.float().cpu() - want).norm() <= 2e-2 * want.norm()


def test_attention_rejects_what_it_cannot_run(cuda_device):
    ra, new = build_pair(128, 64, 2, 1, 256, 1, cuda_device)
    with torch.no_grad():
        with pytest.raises(NotImplementedError):
            new(torch.zeros(1, 8, 128, device=cuda_device))                       # fp32
        with pytest.raises(Exception):
            new(torch.zeros(1, 200, 128, dtype=DT, device=cuda_device))           # context > 128
        with pytest.raises(NotImplementedError):
            new(torch.zeros(2, 8, 128, dtype=DT, device=cuda_device),
                attention_mask=torch.zeros(2, 1, 8, 8, device=cuda_device))        # per-sample masks
