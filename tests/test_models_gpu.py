"""The op inside its three callers: each model restated in monarch_attention_b200/models.py is run
twice on the same seeded weights and inputs - once with the library's attention module, once with a
stand-in that hands q, k, v to the CPU oracle - and the model outputs must agree.  Only the attention
op differs between the two runs, so the comparison is as tight as the op-level one.
(reference call sites: experiments/vit/model.py:93-103, experiments/roberta/model.py:104-106,
experiments/dit/attention_processor.py:131-147)"""
import pytest
import torch

from helpers import error_metrics
from oracle.monarch_oracle import monarch_attention_oracle

pytestmark = pytest.mark.gpu


class OracleAttention(torch.nn.Module):
    """Same call signature as the attention module; the arithmetic happens in the CPU oracle."""

    def __init__(self, block_size, num_steps, pad_type):
        super().__init__()
        self.block_size, self.num_steps, self.pre = block_size, num_steps, pad_type == "pre"

    def forward(self, q, k, v, attention_mask=None):
        m = None if attention_mask is None else attention_mask.cpu()
        out = monarch_attention_oracle(q.cpu().contiguous(), k.cpu().contiguous(), v.cpu().contiguous(), m,
                                       self.num_steps, self.block_size, self.pre)
        return out.to(q.device)


def _both(build, depth, args, attn_args):
    import monarch_attention_b200 as ma
    dev = torch.device("cuda:0")
    outs = []
    for factory in (lambda: ma.MonarchAttention(*attn_args), lambda: OracleAttention(*attn_args)):
        model = build(factory, dtype=torch.bfloat16, device=dev, depth=depth, seed=3)
        with torch.no_grad():
            outs.append(model(*[a.to(dev) for a in args]).float().cpu())
    return outs


def test_vit_b16_with_kernel_matches_vit_with_oracle():
    from monarch_attention_b200.models import build_vit_b16
    g = torch.Generator().manual_seed(0)
    img = torch.rand(2, 3, 224, 224, generator=g).to(torch.bfloat16)
    got, want = _both(build_vit_b16, 2, (img,), (15, 1, "pre"))          # 197 tokens as 14 x 15, front padding
    assert got.shape == (2, 1000)
    assert error_metrics(got.numpy(), want.numpy())[2] < 5e-3


def test_roberta_encoder_with_kernel_matches_encoder_with_oracle():
    from monarch_attention_b200.models import build_roberta_base
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(3, 50265, (4, 512), generator=g)
    mask = torch.ones(4, 512, dtype=torch.long)
    mask[0, 200:] = 0                                                     # right padding: fully masked key blocks
    ids[0, 200:] = 1
    got, want = _both(build_roberta_base, 2, (ids, mask), (32, 1, "post"))
    assert got.shape == (4, 512, 768)
    valid = mask.bool()
    assert error_metrics(got[valid].numpy(), want[valid].numpy())[2] < 5e-3


def test_dit_xl2_with_kernel_matches_dit_with_oracle():
    from monarch_attention_b200.models import build_dit_xl2
    g = torch.Generator().manual_seed(2)
    lat = torch.randn(2, 4, 64, 64, generator=g).to(torch.bfloat16)
    t = torch.randint(0, 1000, (2,), generator=g)
    y = torch.randint(0, 1000, (2,), generator=g)
    got, want = _both(build_dit_xl2, 2, (lat, t, y), (32, 2, "pre"))      # 1024 tokens as 32 x 32, head width 72
    assert got.shape == (2, 8, 64, 64)
    assert error_metrics(got.numpy(), want.numpy())[2] < 5e-3
