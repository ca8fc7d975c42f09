"""Leaf-value functions shared by the CPU and GPU tests of model-valued leaves."""
import torch


def pot_echo_leaf_fn(trees, node_index, hand_weights: torch.Tensor):
    """The function the golden generator's stand-in model computes
    (tests/golden/golden_cfr.py, PotEchoModel) for the tree nodes `node_index` (upstream,
    level-major numbering): s = 0.5 + clamp(pot / (starting_stack_0 + starting_stack_1), 0, 10);
    v0 = s*w + b1; v1 = (s*w)*(-0.5) + b0, every step a separate fp32 operation.  Returns
    fn(beliefs [L,2,1326]) -> values [L,2,1326] evaluated on the device of `beliefs`."""
    st = trees.state
    idx = torch.as_tensor(node_index, dtype=torch.long)
    starting = torch.from_numpy(st.starting_stacks).to(torch.float32)[idx]
    total = starting.sum(dim=1).clamp(min=1.0)
    pot = torch.from_numpy(st.pot).to(torch.float32)[idx]
    frac = (pot / total).clamp_(0.0, 10.0)
    s_host = (0.5 + frac).view(-1, 1)

    def fn(beliefs: torch.Tensor) -> torch.Tensor:
        b = beliefs[..., :1326]
        s = s_host.to(b.device)
        sw = s * hand_weights.to(b.device).view(1, 1326)
        return torch.stack([sw + b[:, 1], sw * (-0.5) + b[:, 0]], dim=1)

    return fn
