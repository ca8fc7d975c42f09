"""Ring buffer for the training batches of the data-generation loop, resident on the device.

Counterpart of the upstream `RebelReplayBuffer` (p2/rl/rebel_replay.py:12-168): the loop adds the
value, pre-chance value and policy batches of every round (`rebel_data_generator.py:80-82`) and the
trainer samples minibatches.  Same insertion order, overwrite rule, optional decimation of
incoming batches once the buffer is full and the same sequence of generator calls, so a buffer fed
the same batches with the same seed holds the same rows.  Batches are `upstream_adapter.RebelBatchLike`
(or anything with its fields); an upstream `RebelBatch` works too, since only attributes are read.
"""
from __future__ import annotations

import torch

from .upstream_adapter import FeatureView, RebelBatchLike

NUM_HANDS = 1326


class ReplayRing:
    def __init__(self, capacity: int, num_actions: int, num_players: int, num_context_features: int, device,
                 policy_targets: bool = True, value_targets: bool = True, dtype: torch.dtype = torch.float32,
                 decimate: float | None = None, generator: torch.Generator | None = None):
        self.capacity, self.num_actions, self.num_players = int(capacity), int(num_actions), int(num_players)
        self.device, self.dtype = torch.device(device), dtype
        self.decimate, self.generator = decimate, generator
        z = lambda *shape, dt=dtype: torch.zeros(*shape, dtype=dt, device=self.device)  # noqa: E731
        self.features = FeatureView(context=z(self.capacity, num_context_features), street=z(self.capacity, dt=torch.long),
                                    to_act=z(self.capacity, dt=torch.long), board=z(self.capacity, 5, dt=torch.long),
                                    beliefs=z(self.capacity, 2 * NUM_HANDS))
        self.policy_targets = z(self.capacity, NUM_HANDS, self.num_actions) if policy_targets else None
        self.value_targets = z(self.capacity, self.num_players, NUM_HANDS) if value_targets else None
        self.legal_masks = z(self.capacity, self.num_actions, dt=torch.bool)
        self.statistics: dict = {}
        self.sample_count = z(self.capacity, dt=torch.long)  # times each row has been sampled
        self.position = 0
        self.size = 0

    def __len__(self) -> int:
        return self.size

    def add_batch(self, batch) -> None:
        """Appends a batch (rebel_replay.py:80-134); a batch longer than the buffer keeps its tail."""
        n = len(batch)
        if n == 0:
            return
        if n >= self.capacity:
            batch = batch[-self.capacity:]
            n = self.capacity
        if (self.policy_targets is None) != (batch.policy_targets is None) or \
                (self.value_targets is None) != (batch.value_targets is None):
            raise ValueError("the batch carries other kinds of targets than the buffer stores")
        if not bool((batch.features.street <= 3).all()):
            raise ValueError("showdown states are never trained on")
        batch = batch.to(self.device)
        if self.decimate is not None and self.size == self.capacity:
            keep = max(1, int(self.decimate * n))
            if keep < n:
                batch = batch[torch.randperm(n, device=self.device, generator=self.generator)[:keep]]
                n = keep
        dest = (torch.arange(n, device=self.device) + self.position) % self.capacity
        f = batch.features
        self.features.context[dest] = f.context.to(self.dtype)
        self.features.street[dest] = f.street.to(torch.long)
        self.features.to_act[dest] = f.to_act.to(torch.long)
        self.features.board[dest] = f.board
        self.features.beliefs[dest] = f.beliefs.to(self.dtype)
        if self.policy_targets is not None:
            self.policy_targets[dest] = batch.policy_targets
        if self.value_targets is not None:
            self.value_targets[dest] = batch.value_targets
        self.legal_masks[dest] = batch.legal_masks
        self.sample_count[dest] = 0
        for key, value in batch.statistics.items():
            if key not in self.statistics:
                self.statistics[key] = torch.zeros(self.capacity, *value.shape[1:], dtype=value.dtype, device=self.device)
            self.statistics[key][dest] = value
        if set(self.statistics) != set(batch.statistics):
            raise ValueError("every batch must carry the same statistics")
        self.position = (self.position + n) % self.capacity
        self.size = min(self.size + n, self.capacity)

    def sample(self, batch_size: int, stratify_streets: list | None = None) -> RebelBatchLike:
        """A minibatch: uniform with replacement, or without replacement with the given probability
        per street (rebel_replay.py:136-181)."""
        if self.size == 0:
            raise ValueError("the replay buffer is empty")
        if batch_size > self.size:
            raise ValueError("cannot take more samples than the buffer holds")
        if stratify_streets is None:
            idx = torch.randint(0, self.size, (batch_size,), generator=self.generator, device=self.device)
        else:
            streets = self.features.street[: self.size]
            weights = torch.tensor(stratify_streets, device=self.device)
            bins = torch.bincount(streets, minlength=4)
            weights[bins == 0] = 0.0
            weights /= weights.sum()
            idx = torch.multinomial((weights / bins)[streets], batch_size, generator=self.generator)
        self.sample_count[idx] += 1
        pick = lambda t: None if t is None else t[idx]  # noqa: E731
        return RebelBatchLike(self.features[idx], self.legal_masks[idx], pick(self.policy_targets),
                              pick(self.value_targets), {k: v[idx] for k, v in self.statistics.items()})

    def clear(self) -> None:
        self.position = 0
        self.size = 0
