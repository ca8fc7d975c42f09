"""A sequence of `RebelReplayBuffer.add_batch` / `sample` calls on seeded batches (upstream
p2/rl/rebel_replay.py), recording the buffer afterwards: wrap-around, a batch longer than the
buffer, decimation once full, uniform and street-stratified sampling.  Imported by make_golden.py."""
from __future__ import annotations

import numpy as np
import torch

import golden_cfr as gc
from golden_cfr import save

SIZES = [5, 7, 3, 20, 6, 4]  # capacity 12: fills, wraps, one oversize batch, then decimated adds


def seeded_batch(n: int, seed: int, num_actions: int = 5):
    """Plain tensors of one value batch; both the generator and the test build the same."""
    g = torch.Generator().manual_seed(seed)
    return dict(
        context=torch.rand(n, 4, generator=g), street=torch.randint(0, 4, (n,), generator=g),
        to_act=torch.randint(0, 2, (n,), generator=g), board=torch.randint(-1, 52, (n, 5), generator=g),
        beliefs=torch.rand(n, 2652, generator=g), legal=torch.rand(n, num_actions, generator=g) > 0.3,
        values=torch.rand(n, 2, 1326, generator=g), pot=torch.randint(1, 500, (n,), generator=g))


def gen_replay() -> None:
    from p2.models.mlp.mlp_features import MLPFeatures
    from p2.rl.rebel_batch import RebelBatch
    from p2.rl.rebel_replay import RebelValueBuffer

    buf = RebelValueBuffer(capacity=12, num_actions=5, num_players=2, num_context_features=4,
                           device=torch.device("cpu"), decimate=0.5, generator=torch.Generator().manual_seed(77))
    for k, n in enumerate(SIZES):
        b = seeded_batch(n, 100 + k)
        buf.add_batch(RebelBatch(features=MLPFeatures(context=b["context"], street=b["street"], to_act=b["to_act"],
                                                      board=b["board"], beliefs=b["beliefs"]),
                                 legal_masks=b["legal"], value_targets=b["values"], statistics={"pot": b["pot"]}))
    uniform = buf.sample(6)
    strat = buf.sample(5, stratify_streets=[0.1, 0.2, 0.3, 0.4])
    save("replay.npz", sizes=np.int64(SIZES), position=np.int64(buf.position), size=np.int64(buf.size),
         context=buf.features.context.numpy(), street=buf.features.street.numpy(), board=buf.features.board.numpy(),
         beliefs_sum=buf.features.beliefs.sum(dim=1).numpy(), values_sum=buf.value_targets.sum(dim=(1, 2)).numpy(),
         legal=buf.legal_masks.numpy(), pot=buf.statistics["pot"].numpy(), sample_count=buf.sample_count.numpy(),
         uniform_pot=uniform.statistics["pot"].numpy(), strat_pot=strat.statistics["pot"].numpy(),
         strat_street=strat.features.street.numpy())


gc.SECTIONS.update(replay=gen_replay)
