"""Chance-node helpers (next-card belief expansion, ordered indexed add) against the CPU
restatement of the upstream helper."""
import pytest
import torch

from oracle import chance as ochance

pytestmark = pytest.mark.gpu


def _setup(seed, B, n_board, L=5):
    g = torch.Generator().manual_seed(seed)
    boards = torch.full((B, L), -1, dtype=torch.int64)
    for b in range(B):
        boards[b, :n_board] = torch.randperm(52, generator=g)[:n_board]
    bel = torch.empty(B, 2, 1326).exponential_(generator=g)
    bel = bel / bel.sum(-1, keepdim=True)
    bel[0, 1] = 0  # empty range -> uniform fallback on every sample
    return boards, bel


@pytest.mark.parametrize("n_board", [3, 4])
def test_expand_next_card(cuda_device, n_board):
    from poker2_b200 import chance

    boards, bel = _setup(3, 5, n_board)
    post, lookup, samples = chance.expand_next_card(bel.to(cuda_device), boards.to(cuda_device))
    epost, elookup, esamples = ochance.expand_next_card(bel, boards)
    assert post.shape[0] == 5 * (52 - n_board)
    assert torch.equal(lookup.cpu(), elookup) and torch.equal(samples.cpu(), esamples)
    torch.testing.assert_close(post.cpu(), epost, rtol=1e-5, atol=1e-9)
    assert torch.equal(post.cpu() == 0, epost == 0)  # exactly the same combos are blocked


def test_indexed_add_rows_ordered_and_ragged(cuda_device):
    from poker2_b200 import chance

    g = torch.Generator().manual_seed(1)
    index = torch.sort(torch.randint(0, 9, (200,), generator=g)).values
    index = index[index != 4]  # row 4 receives nothing
    src = torch.randn(index.numel(), 2, 1326, generator=g)
    out = torch.randn(9, 2, 1326, generator=g)
    want = out.clone().index_add_(0, index, src)
    got = chance.indexed_add_rows(out.to(cuda_device), index.to(cuda_device), src.to(cuda_device))
    assert torch.equal(got.cpu(), want)  # same addition order as the CPU index_add_
    mean = chance.indexed_add_rows(torch.empty(9, 2, 1326, device=cuda_device), index.to(cuda_device),
                                   src.to(cuda_device), mean=True, accumulate=False)
    counts = torch.bincount(index, minlength=9).clamp(min=1).float()
    want_mean = torch.zeros(9, 2, 1326).index_add_(0, index, src) / counts.view(-1, 1, 1)
    assert torch.equal(mean.cpu(), want_mean)
    assert chance.indexed_add_rows(torch.zeros(0, 4, device=cuda_device), torch.zeros(0, dtype=torch.int64,
                                   device=cuda_device), torch.zeros(0, 4, device=cuda_device)).numel() == 0


def test_single_card_chance_values(cuda_device):
    from poker2_b200 import chance

    boards, bel = _setup(9, 4, 4)
    g = torch.Generator().manual_seed(2)
    w = torch.randn(52, generator=g)

    def value_fn(post, samples, lookup):  # a deterministic stand-in for the leaf model
        card = samples[:, 4].to(post.device)
        scale = w.to(post.device)[card].view(-1, 1, 1)
        return torch.stack([post[:, 1], -post[:, 0]], dim=1) * scale + 0.25 * scale

    got = chance.single_card_chance_values(bel.to(cuda_device), boards.to(cuda_device), value_fn)
    want = ochance.single_card_chance_values(bel, boards, value_fn)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-7)
