"""Leaf sampling around the CFR loop: which iteration's policy each root samples from, and the
walk from every root to the public state the next subgame starts at.

Host-side counterpart of `CFREvaluator._get_sampling_schedule`
(p2/search/cfr_evaluator.py:382-404) and `SparseCFREvaluator.sample_leaves`
(p2/search/sparse_cfr_evaluator.py:325-426).  Both draw from a torch generator with the
upstream sequence of calls, so a CPU generator with the same seed gives the same draws.
The tensors they consume come from the solver: `SolveResult.policy_sample` (the policy of
the scheduled iteration, kept by the kernel) and `SolveResult.beliefs_last`.
"""
from __future__ import annotations

import torch

NUM_HANDS = 1326


def sampling_schedule(num_roots: int, iterations: int, generator: torch.Generator | None = None, *,
                      cfr_type: str = "discounted", warm_start_iterations: int = 0, dcfr_delay: int = 0,
                      device=None) -> torch.Tensor:
    """t_sample [num_roots] int64: the iteration at whose start the current policy is kept as
    the sampling policy, drawn with probability proportional to t+1 (uniform for standard
    CFR) from [sample_low, max(iterations, sample_low+1))."""
    if cfr_type == "discounted_plus":
        sample_low = max(warm_start_iterations, dcfr_delay) + 1
    else:
        sample_low = warm_start_iterations + 1
    sample_low = min(sample_low, iterations)
    sample_high = max(iterations, sample_low + 1)
    if cfr_type != "standard":
        distribution = torch.arange(sample_low, sample_high, dtype=torch.float32, device=device) + 1
    else:
        distribution = torch.ones(sample_high - sample_low, device=device)
    distribution /= distribution.sum()
    t_sample = torch.multinomial(distribution, num_roots, replacement=True, generator=generator)
    return t_sample + sample_low


def sample_pass_of(t_sample: torch.Tensor) -> torch.Tensor:
    """The kernel numbers passes by the iteration whose policy they evaluate; the snapshot
    taken at the START of iteration t is the policy of pass t-1."""
    return (t_sample - 1).to(torch.int32)


def _pull_back(trees, x: torch.Tensor) -> torch.Tensor:
    """[top, A, ...] array of the children's rows of x, indexed by (parent, action)."""
    N, M = trees.num_roots, trees.total_nodes
    top = trees.depth_offsets[-2]
    parent = torch.from_numpy(trees.parent_index[N:]).to(x.device)
    action = torch.from_numpy(trees.action_from_parent[N:]).to(x.device)
    out = torch.zeros((top, trees.num_actions, *x.shape[1:]), dtype=x.dtype, device=x.device)
    out[parent, action] = x[N:M]
    return out


def sample_leaves(trees, policy_sample: torch.Tensor, beliefs: torch.Tensor, generator: torch.Generator | None = None,
                  *, sample_epsilon: float = 0.25, training_mode: bool = True):
    """Walks from every root to a leaf, the walking hand drawn from the root's acting-player
    beliefs and actions from `policy_sample` (uniform with probability `sample_epsilon` at the
    nodes of one randomly chosen player), never stepping into a finished hand.

    trees: `tree.PublicTrees`; policy_sample [M,1326] and beliefs [M,2,1326] in the upstream
    (level-major) node order.  Returns (sampled_nodes [N], continue_nodes, beliefs[continue_nodes]):
    continue_nodes are the sampled nodes that are not roots, the public states the next
    subgames start from."""
    device = policy_sample.device
    N = trees.num_roots
    top = trees.depth_offsets[-2]
    st = trees.state
    to_act = torch.from_numpy(st.to_act).to(device)
    done = torch.from_numpy(st.done).to(device)
    leaf_mask = torch.from_numpy(trees.leaf_mask).to(device)
    child_mask = torch.from_numpy(trees.legal_mask & ~trees.leaf_mask[:, None]).to(device)
    child_offsets = torch.from_numpy(trees.child_offsets).to(device)

    players = torch.randint(0, 2, (N,), generator=generator, device=device)
    eps = sample_epsilon if training_mode else 0.0
    done_src = _pull_back(trees, done)
    sampling_masks = child_mask.clone()
    sampling_masks[:top] &= ~done_src
    sampling_counts = sampling_masks.float().sum(dim=-1, keepdim=True)
    uniform = torch.where(sampling_masks, 1 / sampling_counts, 0)
    by_src = _pull_back(trees, policy_sample).clone()
    by_src.masked_fill_(done_src[:, :, None], 0.0)
    denom = by_src.sum(dim=1, keepdim=True)
    by_src = torch.where(denom >= 1e-12, by_src / denom, uniform[:top, :, None])
    child_action_index = child_mask.int().cumsum(dim=1) - child_mask.int()
    effective_leaf = leaf_mask | (sampling_counts.squeeze(1) == 0)

    actor_beliefs = beliefs[:N].gather(1, to_act[:N, None, None].expand(-1, -1, beliefs.shape[-1])).squeeze(1)
    hands = torch.multinomial(actor_beliefs, 1, generator=generator).squeeze(1)
    nodes = torch.arange(N, device=device)
    active = ~effective_leaf[nodes]
    while active.any():
        act_nodes = nodes[active]
        count = act_nodes.numel()
        uniformly = torch.rand(count, generator=generator, device=device) < eps
        uniformly &= to_act[act_nodes] == players[active]
        probs = by_src[act_nodes, :, hands[active]]
        actions = torch.multinomial(torch.where(uniformly[:, None], uniform[act_nodes], probs), num_samples=1,
                                    generator=generator).squeeze(1)
        nodes[active] = child_offsets[act_nodes] + child_action_index[act_nodes, actions]
        active = ~effective_leaf[nodes]
    cont = nodes[nodes >= N]
    return nodes, cont, beliefs[cont]
