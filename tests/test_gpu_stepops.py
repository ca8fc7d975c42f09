"""Step-level kernels (the `fused_cfr_triton` call signatures) against torch restatements
of the upstream op sequences they replace, on real ragged trees."""
import numpy as np
import pytest
import torch

from oracle import unblocked as ounblocked
from poker2_b200 import tree as ptree

pytestmark = pytest.mark.gpu
H = 1326
RTOL, ATOL = 1e-5, 1e-6


@pytest.fixture(scope="module")
def T(cuda_device):
    pot = np.array([100, 40, 180]); stack = np.array([400, 900, 150])
    t = ptree.build_trees(ptree.root_states(pot, stack), [0.5, 1.0], 8, max_raises=2)
    dev = cuda_device
    g = torch.Generator().manual_seed(0)
    M, N, top = t.total_nodes, t.num_roots, t.depth_offsets[-2]
    d = dict(
        M=M, N=N, top=top, offs=t.depth_offsets, dev=dev, g=g,
        parent=torch.from_numpy(t.parent_index), prev_actor=torch.from_numpy(t.prev_actor),
        to_act=torch.from_numpy(t.state.to_act), child_count=torch.from_numpy(t.child_count),
        child_offsets=torch.from_numpy(t.child_offsets), root_of=torch.from_numpy(t.root_of),
    )
    return d


def rnd(T, *shape, positive=True):
    x = torch.rand(*shape, generator=T["g"])
    return x if positive else x - 0.5


def cu(T, x):
    return x.to(T["dev"]).contiguous()


def test_dcfr_update(T):
    from poker2_b200 import fused_cfr as F

    class Kind:
        name = "discounted"

    c, w, r = rnd(T, 50, H, positive=False), rnd(T, 50, H), rnd(T, 50, H, positive=False)
    for t, plus in ((0, False), (7, False), (3, True)):
        cg, wg, rg, pos = cu(T, c), cu(T, w), cu(T, r), torch.empty(50, H, device=T["dev"])
        F.fused_dcfr_update_(cg, wg, rg, t, Kind, 1.5, 0.0, plus, positive_regrets_out=pos)
        num = torch.where(c > 0, t ** 1.5, t ** 0.0); den = torch.where(c > 0, t ** 1.5 + 1, t ** 0.0 + 1)
        ce = c.clone(); ce *= num; ce /= den; we = w.clone(); we *= num; we /= den
        we += 1; ce += r
        if plus: ce.clamp_(min=0)
        assert torch.equal(cg.cpu(), ce) and torch.equal(wg.cpu(), we) and torch.equal(pos.cpu(), ce.clamp(min=0))


def test_block_normalize_and_deep_beliefs(T):
    from poker2_b200 import fused_cfr as F

    M, N = T["M"], T["N"]
    allowed = torch.rand(M, H, generator=T["g"]) > 0.2
    prob = allowed.float() / allowed.float().sum(-1, keepdim=True)
    x = rnd(T, M, 2, H); x[3] = 0  # an empty row takes the fallback
    xg = cu(T, x)
    F.fused_block_and_normalize_beliefs_(xg, cu(T, allowed), cu(T, prob))
    e = x.masked_fill((~allowed)[:, None, :], 0.0); s = e.sum(-1, keepdim=True)
    e = torch.where(s > 1e-5, e / s, prob[:, None, :])
    torch.testing.assert_close(xg.cpu(), e, rtol=RTOL, atol=ATOL)

    reach = rnd(T, M, 2, H) * allowed[:, None, :]; reach[N + 2, 1] = 0
    out = cu(T, rnd(T, M, 2, H)); roots = out[:N].clone().cpu()
    F.fused_deep_beliefs_(out, out, cu(T, reach), cu(T, prob), cu(T, T["root_of"]), num_roots=N)
    v = roots[T["root_of"]] * reach; s = v.sum(-1, keepdim=True)
    e = torch.where(s > 1e-5, v / s, prob[:, None, :])
    torch.testing.assert_close(out.cpu()[N:], e[N:], rtol=RTOL, atol=ATOL)
    assert torch.equal(out.cpu()[:N], roots)


def test_policy_steps(T):
    from poker2_b200 import fused_cfr as F

    M, N, top = T["M"], T["N"], T["top"]
    par, cc, co = T["parent"], T["child_count"], T["child_offsets"]
    regrets = rnd(T, M, H, positive=False); regrets[N + 1: N + 3] = -1.0  # all-negative siblings -> fallback path
    pos = regrets.clamp(min=0.0)
    psum = F.fused_parent_sum(cu(T, pos), cu(T, co[:top]), cu(T, cc[:top]), max_children=5)
    e = torch.zeros(top, H); e.index_add_(0, par[N:], pos[N:])
    torch.testing.assert_close(psum.cpu(), e, rtol=RTOL, atol=ATOL)
    sib = F.fused_sibling_sum(cu(T, pos), cu(T, co[:top]), cu(T, cc[:top]), N, M - N, max_children=5)
    torch.testing.assert_close(sib.cpu(), e[par[N:]], rtol=RTOL, atol=ATOL)
    uniform = (1.0 / cc[par[N:]].float())[:, None].expand(-1, H).contiguous()
    out = torch.empty(M - N, H, device=T["dev"])
    F.fused_divide_by_parent_sum_(cu(T, pos[N:]), cu(T, uniform), psum, cu(T, par[N:]), out)
    den = psum.cpu()[par[N:]]
    want = torch.where(den > 1e-8, pos[N:] / den.clamp(min=1e-8), uniform)
    assert torch.equal(out.cpu(), want)
    out2 = torch.empty_like(out)
    F.fused_regret_matching_divide_(cu(T, pos[N:]), cu(T, den), cu(T, uniform), out2)
    assert torch.equal(out2.cpu(), want)

    reach, reach_avg = rnd(T, M, 2, H), rnd(T, M, 2, H); reach[0] = 0; reach_avg[0] = 0
    pol, avg = rnd(T, M, H), rnd(T, M, H)
    avg_g = cu(T, avg)
    F.fused_average_policy_mix_(avg_g, cu(T, pol), cu(T, reach), cu(T, reach_avg), cu(T, T["to_act"]), cu(T, par),
                                old=9.0, new=16.0, bottom=N)
    idx = T["to_act"][:top, None, None].expand(-1, -1, H)
    ra = reach_avg[:top].gather(1, idx).squeeze(1) * 9.0; rn = reach[:top].gather(1, idx).squeeze(1) * 16.0
    ra, rn = ra[par[N:]], rn[par[N:]]
    num = ra * avg[N:] + rn * pol[N:]; dn = ra + rn
    plain = (9.0 * avg[N:] + 16.0 * pol[N:]) / 25.0
    assert torch.equal(avg_g.cpu()[N:], torch.where(dn > 1e-5, num / dn, plain))
    assert torch.equal(avg_g.cpu()[:N], avg[:N])


def test_value_steps(T):
    from poker2_b200 import fused_cfr as F

    M, N, top, offs = T["M"], T["N"], T["top"], T["offs"]
    par, pa, cc, co = T["parent"], T["prev_actor"].clamp(min=0), T["child_count"], T["child_offsets"]
    vals, hero, opp = rnd(T, M, 2, H, positive=False), rnd(T, M, H), rnd(T, M, H)
    out = torch.empty(M, 2, H, device=T["dev"])
    F.fused_weight_child_values(cu(T, vals), cu(T, pa), cu(T, hero), cu(T, opp), out)
    w = vals.clone(); rows = torch.arange(M)
    w[rows, pa] *= hero; w[rows, 1 - pa] *= opp
    assert torch.equal(out.cpu(), w)

    vg = cu(T, vals)
    for d in range(len(offs) - 3, -1, -1):
        a, b = offs[d], offs[d + 1]
        F.fused_weighted_parent_sum(vg, cu(T, T["prev_actor"]), cu(T, hero), cu(T, opp), cu(T, co[a:b]), cu(T, cc[a:b]),
                                    parent_base=a, max_children=5)
    e = vals.clone()
    for d in range(len(offs) - 3, -1, -1):
        a, b, c = offs[d], offs[d + 1], offs[d + 2]
        ww = e[b:c].clone(); r = torch.arange(c - b); p = T["prev_actor"][b:c]
        ww[r, p] *= hero[b:c]; ww[r, 1 - p] *= opp[b:c]
        acc = torch.zeros(b - a, 2, H); acc.index_add_(0, par[b:c] - a, ww)
        nonleaf = cc[a:b] > 0
        e[a:b][nonleaf] = acc[nonleaf]
    torch.testing.assert_close(vg.cpu(), e, rtol=RTOL, atol=ATOL)

    regrets = torch.zeros(M, H, device=T["dev"])
    av, sw = rnd(T, top, H, positive=False), rnd(T, top, H)
    F.fused_regret_tail_(regrets, cu(T, vals), cu(T, av), cu(T, sw), cu(T, par), cu(T, T["prev_actor"]), bottom=N)
    ach = vals[N:].gather(1, T["prev_actor"][N:, None, None].expand(-1, -1, H)).squeeze(1)
    assert torch.equal(regrets.cpu()[N:], sw[par[N:]] * (ach - av[par[N:]]))

    a0, lat, bel = rnd(T, M, 2, H, positive=False), rnd(T, M, 2, H, positive=False), rnd(T, M, 2, H)
    ag = cu(T, a0)
    F.fused_update_average_values_(ag, cu(T, lat), old=4.0, new=9.0)
    mixed = (a0 * 4.0 + lat * 9.0) * torch.tensor(1.0 / 13.0)
    torch.testing.assert_close(ag.cpu(), mixed, rtol=RTOL, atol=ATOL)
    S = F.TScalars(T["dev"]); S.update(3, 1.5, 0.0, 4.0, 9.0)
    ignore = torch.rand(M, generator=T["g"]) > 0.7
    ag = cu(T, a0)
    F.fused_avg_values_zero_sum_(ag, cu(T, lat), cu(T, bel), S.mix_old, S.mix_new, S.mix_inv_total, True,
                                 ignore_mask=cu(T, ignore))
    shift = (mixed * bel).sum(dim=2, keepdim=True).mean(dim=1, keepdim=True).masked_fill(ignore[:, None, None], 0.0)
    torch.testing.assert_close(ag.cpu(), mixed - shift, rtol=1e-4, atol=1e-5)
    got = F.fused_model_values_mix(cu(T, a0), cu(T, lat), old=4.0, new=9.0)
    torch.testing.assert_close(got.cpu(), ((4.0 + 9.0) * a0 - 4.0 * lat) / 9.0, rtol=1e-5, atol=1e-5)
    outz = torch.empty(M, 2, H, device=T["dev"])
    F.fused_model_values_mix_zero_sum(cu(T, a0), cu(T, lat), cu(T, bel), S.mix_onon, S.mix_oon, outz, True)
    u = a0 * (13.0 / 9.0) - lat * (4.0 / 9.0)
    torch.testing.assert_close(outz.cpu(), u - (u * bel).sum(2, keepdim=True).mean(1, keepdim=True), rtol=1e-4, atol=1e-5)


def test_reach_and_unblocked(T):
    from poker2_b200 import fused_cfr as F

    M, N, top, offs = T["M"], T["N"], T["top"], T["offs"]
    par, pa = T["parent"], T["prev_actor"]
    allowed = torch.rand(M, H, generator=T["g"]) > 0.1
    pol = rnd(T, M, H)
    reach = torch.zeros(M, 2, H); reach[:N] = 1.0
    rg = cu(T, reach)
    for d in range(len(offs) - 2):
        F.fused_reach_weights_depth_(rg, cu(T, pol), cu(T, allowed), cu(T, par), cu(T, pa), offs[d + 1], offs[d + 2])
    e = reach.clone()
    for d in range(len(offs) - 2):
        b, c = offs[d + 1], offs[d + 2]
        e[b:c] = e[par[b:c]]
        e[torch.arange(b, c), pa[b:c]] *= pol[b:c]
        e[b:c] = e[b:c] * allowed[b:c][:, None, :]
    assert torch.equal(rg.cpu(), e)

    x = rnd(T, 7, 2, H); x[2] = 0; x[2, 0, 17] = 1.0
    got = F.unblocked_mass_triton(cu(T, x))
    torch.testing.assert_close(got.cpu(), ounblocked.unblocked_mass(x), rtol=1e-6, atol=1e-7)
    bel = rnd(T, M, 2, H)
    got = F.unblocked_mass_opp_at_parents_triton(cu(T, bel), cu(T, T["to_act"]), top)
    opp = bel[:top].gather(1, (1 - T["to_act"][:top])[:, None, None].expand(-1, -1, H)).squeeze(1)
    torch.testing.assert_close(got.cpu(), ounblocked.unblocked_mass(opp), rtol=1e-6, atol=1e-7)
    actor = rnd(T, top, H); actor[1] = 0  # zero denominator -> ratio 0
    marg = actor[par[N:]] * pol[N:]
    got = F.unblocked_mass_ratio_indirect_triton(cu(T, marg), cu(T, actor), cu(T, par[N:]))
    un, ud = ounblocked.unblocked_mass(marg), ounblocked.unblocked_mass(actor)[par[N:]]
    want = torch.where(ud > 1e-5, un / ud, torch.zeros(()))
    torch.testing.assert_close(got.cpu(), want, rtol=RTOL, atol=ATOL)
    got = F.unblocked_mass_ratio_triton(cu(T, marg), cu(T, actor[par[N:]]))
    torch.testing.assert_close(got.cpu(), want, rtol=RTOL, atol=ATOL)
