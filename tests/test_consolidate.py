"""ModuleList experts -> fused tensors (scattermoe_b200.utils.consolidate): the copy, the memory release, and
checkpoints that keep the per-expert key layout in both directions. Host only; the forward is checked on the GPU
(tests/test_gpu_mlp.py::test_consolidated_module_list_block)."""
import pytest
import torch
from torch import nn

from scattermoe_b200.utils import consolidate as C


class ExpertMLP(nn.Module):
    def __init__(self, hidden, inter, names=C.QWEN_NAMES):
        super().__init__()
        g, u, d = names
        setattr(self, g, nn.Linear(hidden, inter, bias=False))
        setattr(self, u, nn.Linear(hidden, inter, bias=False))
        setattr(self, d, nn.Linear(inter, hidden, bias=False))
        self.act_fn = nn.SiLU()


class Block(nn.Module):
    def __init__(self, hidden=16, inter=24, E=4, names=C.QWEN_NAMES):
        super().__init__()
        self.gate = nn.Linear(hidden, E, bias=False)
        self.experts = nn.ModuleList([ExpertMLP(hidden, inter, names) for _ in range(E)])
        self.top_k, self.norm_topk_prob = 2, True


@pytest.mark.parametrize("names", [C.QWEN_NAMES, C.MIXTRAL_NAMES])
def test_consolidation_copies_every_expert_and_releases_the_originals(names):
    torch.manual_seed(0)
    block = Block(names=names)
    before = {k: v.clone() for k, v in block.state_dict().items()}
    originals = block.experts
    C.consolidate_moe_block(block, names=names)
    fused = block.experts
    assert isinstance(fused, C.ConsolidatedExperts)
    assert fused.gate_up_proj.shape == (4, 48, 16) and fused.down_proj.shape == (4, 16, 24)
    assert fused.gate_up_proj.requires_grad and isinstance(fused.act_fn, nn.SiLU)
    g, u, d = names
    for i in range(4):
        assert torch.equal(fused.gate_up_proj[i, :24], before["experts.%d.%s.weight" % (i, g)])
        assert torch.equal(fused.gate_up_proj[i, 24:], before["experts.%d.%s.weight" % (i, u)])
        assert torch.equal(fused.down_proj[i], before["experts.%d.%s.weight" % (i, d)])
        assert all(p.numel() == 0 for p in originals[i].parameters()), "the expert's storage must have been released"
    # idempotent
    assert C.consolidate_moe_block(block, names=names).experts is fused


def test_state_dict_keeps_the_per_expert_layout_both_ways():
    torch.manual_seed(1)
    plain = Block()
    want = {k: v.clone() for k, v in plain.state_dict().items()}
    fused_block = C.consolidate_moe_block(Block())
    # load a per-expert checkpoint into the consolidated block (strict): merged on the way in
    missing, unexpected = fused_block.load_state_dict(want, strict=True)
    assert not missing and not unexpected
    # save: split on the way out, same keys, same values
    got = fused_block.state_dict()
    assert sorted(got) == sorted(want)
    for k in want:
        assert torch.equal(got[k], want[k]), k
    # and the saved checkpoint loads into an un-consolidated block
    fresh = Block()
    fresh.load_state_dict(got, strict=True)
    # a fused checkpoint (keys gate_up_proj / down_proj) is accepted as well
    fused_keys = {"gate.weight": want["gate.weight"], "experts.gate_up_proj": fused_block.experts.gate_up_proj.detach().clone(),
                  "experts.down_proj": fused_block.experts.down_proj.detach().clone()}
    other = C.consolidate_moe_block(Block())
    other.load_state_dict(fused_keys, strict=True)
    assert torch.equal(other.experts.down_proj, fused_block.experts.down_proj)


def test_incomplete_checkpoint_is_reported():
    block = C.consolidate_moe_block(Block())
    sd = Block().state_dict()
    del sd["experts.2.up_proj.weight"]
    with pytest.raises(RuntimeError, match="lacks experts.2.up_proj.weight"):
        block.load_state_dict(sd, strict=True)


def test_rejects_experts_it_cannot_fuse():
    block = Block()
    block.experts[0].gate_proj = nn.Linear(16, 24, bias=True)
    with pytest.raises(AssertionError, match="bias-free"):
        C.consolidate_experts(block.experts)
    with pytest.raises(AssertionError, match="empty"):
        C.consolidate_experts(nn.ModuleList())
