"""Public betting trees for a batch of subgames (host side, numpy).

Builds what `SparseCFREvaluator._construct_subgame` builds
(p2/search/sparse_cfr_evaluator.py:141-306) with the betting rules of `HUNLTensorEnv`
(p2/env/hunl_tensor_env.py: `legal_bins_amounts_and_mask` :348-423, `step` :766-992,
`finish_and_assign_rewards` :707-724): breadth-first expansion of every legal bet bin,
one level at a time over the whole batch, stopping at terminal nodes, at the start of a new
street and at `max_depth`.  Node order, parent indices, action indices and legal masks are
bit-identical to the upstream arrays.  `max_raises` (not an upstream option) additionally
removes the bet/raise/all-in bins once that many have been made on the street.

Two layouts are offered: the upstream level-major order over the batch (`PublicTrees`
fields), and a subgame-major order with 16-byte node records for the CUDA solver
(`DeviceTreeLayout`).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

KIND_INTERNAL, KIND_FOLD, KIND_SHOWDOWN, KIND_MODEL = 0, 1, 2, 3
MAX_NODES_PER_SUBGAME = 255
MAX_CHILDREN = 8


@dataclass
class RoundState:
    """Betting state of a batch of public nodes (all int64 / bool arrays of length n)."""

    to_act: np.ndarray
    pot: np.ndarray
    stacks: np.ndarray  # [n,2]
    committed: np.ndarray  # [n,2]
    min_raise: np.ndarray
    actions_this_round: np.ndarray
    is_allin: np.ndarray  # [n,2] bool
    done: np.ndarray  # bool
    street: np.ndarray  # 0..4, 4 = showdown reached
    button: np.ndarray
    starting_stacks: np.ndarray  # [n,2]
    scale: np.ndarray  # fp32
    raises: np.ndarray  # bets/raises/all-ins made on this street

    def take(self, idx: np.ndarray) -> "RoundState":
        return RoundState(**{k: v[idx].copy() for k, v in self.__dict__.items()})

    @property
    def n(self) -> int:
        return self.to_act.shape[0]


def root_states(pot, stacks, *, to_act=None, button=None, street=3, min_raise=2, starting_stacks=None,
                scale=None) -> RoundState:
    """States at the start of a betting round.  `starting_stacks` defaults to
    stacks + pot/2 (both players put in half the pot) and `scale` to starting_stacks[:,0],
    the conventions of the upstream environment (hunl_tensor_env.py:293-296)."""
    pot = np.asarray(pot, dtype=np.int64)
    n = pot.shape[0]
    stacks = np.asarray(stacks, dtype=np.int64)
    if stacks.ndim == 1:
        stacks = np.stack([stacks, stacks], axis=1)
    button = np.zeros(n, dtype=np.int64) if button is None else np.asarray(button, dtype=np.int64)
    to_act = (1 - button) if to_act is None else np.asarray(to_act, dtype=np.int64)
    if starting_stacks is None:
        starting_stacks = stacks + (pot // 2)[:, None]
    starting_stacks = np.asarray(starting_stacks, dtype=np.int64)
    if scale is None:
        scale = starting_stacks[:, 0].astype(np.float32)
    z = np.zeros(n, dtype=np.int64)
    return RoundState(
        to_act=to_act.copy(), pot=pot.copy(), stacks=stacks.copy(), committed=np.zeros((n, 2), dtype=np.int64),
        min_raise=np.full(n, min_raise, dtype=np.int64) if np.isscalar(min_raise) else np.asarray(min_raise, np.int64),
        actions_this_round=z.copy(), is_allin=np.zeros((n, 2), dtype=bool), done=np.zeros(n, dtype=bool),
        street=np.full(n, street, dtype=np.int64) if np.isscalar(street) else np.asarray(street, np.int64),
        button=button.copy(), starting_stacks=starting_stacks.copy(), scale=np.asarray(scale, dtype=np.float32),
        raises=z.copy(),
    )


def legal_bins(s: RoundState, bet_bins, max_raises=None):
    """(amounts [n,A], mask [n,A]) of the bins {fold, check/call, pot fractions..., all-in}
    (hunl_tensor_env.py:348-423)."""
    n, A = s.n, len(bet_bins) + 3
    rows = np.arange(n)
    me, opp = s.to_act, 1 - s.to_act
    me_stack, opp_stack = s.stacks[rows, me], s.stacks[rows, opp]
    to_call = s.committed[rows, opp] - s.committed[rows, me]
    amounts = np.full((n, A), -1, dtype=np.int64)
    mask = np.zeros((n, A), dtype=bool)
    mask[:, 0] = to_call > 0
    mask[:, 1] = True
    frac = np.asarray(bet_bins, dtype=np.float32)[None, :]
    extra = (frac * s.pot.astype(np.float32)[:, None]).astype(np.int64)  # fp32 product, truncated
    raise_to = to_call[:, None] + extra
    ok = ((me_stack > 0) & (opp_stack > 0))[:, None] & (raise_to <= me_stack[:, None]) & (extra >= s.min_raise[:, None])
    amounts[:, 2:-1] = raise_to
    mask[:, 2:-1] = ok
    amounts[:, A - 1] = me_stack
    mask[:, A - 1] = me_stack > 0
    opp_allin = s.is_allin[rows, opp]
    mask[opp_allin, 0:2] = True
    mask[opp_allin, 2:] = False
    me_allin = s.is_allin[rows, me]
    mask[me_allin, :] = False
    mask[me_allin, 1] = True
    mask &= ~s.done[:, None]
    if max_raises is not None:
        mask[:, 2:] &= (s.raises < max_raises)[:, None]
    return amounts, mask


def step(s: RoundState, bins: np.ndarray, amounts: np.ndarray, num_bins: int, bb) -> np.ndarray:
    """Applies one bin per node in place; returns the fp32 reward of player 0 at nodes that
    ended by a fold (hunl_tensor_env.py:766-992, 707-724)."""
    n = s.n
    rows = np.arange(n)
    actor, other = s.to_act.copy(), 1 - s.to_act
    actor_stack = s.stacks[rows, actor]
    to_call = s.committed[rows, other] - s.committed[rows, actor]
    rewards = np.zeros(n, dtype=np.float32)

    fold = bins == 0
    if fold.any():
        s.done[fold] = True
        winner0 = other[fold] == 0
        pot_f = s.pot[fold].astype(np.float32)
        share = np.where(winner0, pot_f, np.float32(0.0)).astype(np.float32)
        num = s.stacks[fold, 0].astype(np.float32) + share - s.starting_stacks[fold, 0].astype(np.float32)
        rewards[fold] = (num / s.scale[fold]).astype(np.float32)

    chips = np.zeros(n, dtype=np.int64)
    call = bins == 1
    chips[call] = np.minimum(to_call[call], actor_stack[call])
    allin = bins == num_bins - 1
    chips[allin] = actor_stack[allin]
    bet = (bins >= 2) & (bins < num_bins - 1)
    chips[bet] = amounts[rows[bet], bins[bet]]
    s.stacks[rows, actor] -= chips
    s.committed[rows, actor] += chips
    s.pot += chips
    s.is_allin[rows[allin], actor[allin]] = True
    s.min_raise[bet] = np.maximum(s.min_raise[bet], chips[bet] - to_call[bet])
    s.raises += (bins >= 2).astype(np.int64)

    s.to_act[:] = 1 - actor
    s.actions_this_round += 1

    c0, c1 = s.committed[:, 0], s.committed[:, 1]
    a0, a1 = s.is_allin[:, 0], s.is_allin[:, 1]
    closed = (~s.done) & ((c0 == c1) | (a0 & a1) | (a0 & (c0 <= c1)) | (a1 & (c1 <= c0))) & (s.actions_this_round >= 2)
    if closed.any():
        s.committed[closed] = 0
        s.actions_this_round[closed] = 0
        s.to_act[closed] = 1 - s.button[closed]
        s.min_raise[closed] = np.asarray(bb, dtype=np.int64)[closed] if np.ndim(bb) else bb
        s.raises[closed] = 0
        river = closed & (s.street == 3)
        s.done[river] = True  # showdown; its value comes from the range-vs-range evaluator
        s.street[closed] += 1
    return rewards


@dataclass
class PublicTrees:
    """A batch of public trees in the upstream node order."""

    num_roots: int
    num_actions: int
    depth_offsets: list
    parent_index: np.ndarray
    action_from_parent: np.ndarray
    state: RoundState  # all nodes
    legal_mask: np.ndarray  # [M,A]
    leaf_mask: np.ndarray
    new_street_mask: np.ndarray
    child_count: np.ndarray
    child_offsets: np.ndarray
    prev_actor: np.ndarray
    fold_value: np.ndarray  # fp32, value of player 0 at fold leaves
    showdown_potential: np.ndarray  # [M,2] int64 (meaningful where street == 4)
    root_of: np.ndarray
    depth_of: np.ndarray
    extra: dict = field(default_factory=dict)

    @property
    def total_nodes(self) -> int:
        return self.depth_offsets[-1]

    @property
    def tree_depth(self) -> int:
        return len(self.depth_offsets) - 2

    def oracle_dict(self, boards) -> dict:
        """The arrays the CPU oracle consumes (see oracle/cfr.py)."""
        return dict(
            depth_offsets=np.asarray(self.depth_offsets, dtype=np.int64), parent_index=self.parent_index,
            action_from_parent=self.action_from_parent, to_act=self.state.to_act, child_count=self.child_count,
            leaf_mask=self.leaf_mask, done=self.state.done, street=self.state.street, fold_value=self.fold_value,
            showdown_potential=self.showdown_potential, scale=self.state.scale, boards=np.asarray(boards),
            num_actions=self.num_actions,
        )


def _concat_states(levels) -> RoundState:
    return RoundState(**{k: np.concatenate([getattr(l, k) for l in levels]) for k in levels[0].__dict__})


def build_trees(roots: RoundState, bet_bins, max_depth: int, *, bb=2, max_raises=None) -> PublicTrees:
    A = len(bet_bins) + 3
    n_roots = roots.n
    levels = [roots.take(np.arange(n_roots))]
    parents = [np.full(n_roots, -1, dtype=np.int64)]
    actions = [np.full(n_roots, -1, dtype=np.int64)]
    rewards = [np.zeros(n_roots, dtype=np.float32)]
    offs = [0, n_roots]
    depth = 0
    while depth < max_depth:
        cur = levels[-1]
        amounts, mask = legal_bins(cur, bet_bins, max_raises)
        if depth > 0:
            mask &= (cur.actions_this_round != 0)[:, None]
        rows_idx, bins = np.nonzero(mask)
        if bins.size == 0:
            break
        nxt = cur.take(rows_idx)
        if np.ndim(bb):  # one big blind per root: carried down the levels with the nodes
            bb_level = np.asarray(bb, dtype=np.int64) if depth == 0 else bb_level
            bb_level = bb_level[rows_idx]
        bb_rows = bb_level if np.ndim(bb) else bb
        rew = step(nxt, bins, amounts[rows_idx], A, bb_rows)
        levels.append(nxt)
        parents.append(offs[-2] + rows_idx)
        actions.append(bins.astype(np.int64))
        rewards.append(rew)
        depth += 1
        offs.append(offs[-1] + nxt.n)

    state = _concat_states(levels)
    M = offs[-1]
    parent_index = np.concatenate(parents)
    action = np.concatenate(actions)
    reward = np.concatenate(rewards)
    _, legal = legal_bins(state, bet_bins, max_raises)
    is_root = np.zeros(M, dtype=bool)
    is_root[:n_roots] = True
    new_street = (state.actions_this_round == 0) & ~is_root
    leaf = state.done | new_street
    leaf[offs[-2]:] = True
    child_mask = legal & ~leaf[:, None]
    child_count = child_mask.sum(axis=1).astype(np.int64)
    assert M == n_roots + child_count.sum(), "tree bookkeeping mismatch"
    child_offsets = n_roots + np.cumsum(child_count) - child_count
    prev_actor = np.full(M, -1, dtype=np.int64)
    prev_actor[n_roots:] = state.to_act[parent_index[n_roots:]]
    folded = (action == 0) & state.done
    fold_value = np.where(folded, reward, np.float32(0)).astype(np.float32)
    potential = state.stacks + state.pot[:, None] - state.starting_stacks
    root_of = np.arange(M)
    depth_of = np.zeros(M, dtype=np.int64)
    for d in range(len(offs) - 2):
        a, b = offs[d + 1], offs[d + 2]
        root_of[a:b] = root_of[parent_index[a:b]]
        depth_of[a:b] = d + 1
    return PublicTrees(
        num_roots=n_roots, num_actions=A, depth_offsets=offs, parent_index=parent_index, action_from_parent=action,
        state=state, legal_mask=legal, leaf_mask=leaf, new_street_mask=new_street, child_count=child_count,
        child_offsets=child_offsets, prev_actor=prev_actor, fold_value=fold_value, showdown_potential=potential,
        root_of=root_of, depth_of=depth_of,
    )
