"""The mixture-of-experts glue around the expert GEMMs: the shared expert's sigmoid gate (zero/kernels/moe.cl:44,88,344-352)
and the expert-parallel split (zero/mgpu/engine_tp_shard.h:169-199, zero/kernels/tp.cl:55-111), against the oracle: routing,
slots and tiles exact, the combine bit for bit (it has a defined order), the split sum against the unsplit one."""
import numpy as np
import pytest

from arcinferzero_b200 import synth as S
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch as t
    assert t.cuda.is_available()
    return t


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_shared_expert_gate_and_combine(izb, torch):
    rng = np.random.default_rng(1)
    T, NE, NU, E = 333, 60, 4, 256
    lg = rng.standard_normal((T, NE + 1)).astype(np.float32) * 3
    ids, wts, counts, sgate = izb.moe_route(dev(torch, lg), NU, shared_gate=True)
    rid, rwt, rcnt = O.moe_route(np.ascontiguousarray(lg[:, :NE]), NU)
    assert (ids.cpu().numpy() == rid).all() and (counts.cpu().numpy() == rcnt).all()
    assert np.abs(sgate.cpu().numpy() - O.moe_sgate(lg, NE)).max() <= 1e-6
    offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, 8)
    y = rng.standard_normal((T * NU, E)).astype(np.float32)
    sh = rng.standard_normal((T, E)).astype(np.float32)
    x = rng.standard_normal((T, E)).astype(np.float32)
    out = dev(torch, x)
    izb.moe_combine(out, dev(torch, y), inv, NU, sh=dev(torch, sh), sgate=sgate)
    ref = O.moe_combine_ex(x, y, inv.cpu().numpy(), NU, sh=sh, sgate=sgate.cpu().numpy())
    assert (bits(out.cpu().numpy()) == bits(ref)).all()


def test_expert_parallel_split_adds_up(izb, torch):
    """Two ranks' worth of experts run one after the other on one GPU: each sorts only its own (token, expert) pairs, runs
    its expert GEMMs on its own stack, and combines into a partial output; residual + partials (tp_add, rank order) must
    equal the unsplit block."""
    rng = np.random.default_rng(2)
    T, E, F, NE, NU, qt, TM = 200, 512, 256, 8, 3, 12, 8
    wg, wu = S.make_weight(qt, NE * F, E, 11), S.make_weight(qt, NE * F, E, 12)
    wd = S.make_weight(qt, NE * E, F, 13)
    x = S.make_act(T, E, 14)
    lg = rng.standard_normal((T, NE + 1)).astype(np.float32)
    sh = rng.standard_normal((T, E)).astype(np.float32)
    Tp = izb.pad_rows(T)
    aq, asc, _ = izb.quantize_act(dev(torch, x), Mp=Tp)
    ids, wts, counts, sgate = izb.moe_route(dev(torch, lg), NU, shared_gate=True)
    Sn = T * NU
    Sp = izb.pad_rows(Sn)

    def run(e0, e1, shared):
        n = e1 - e0
        Wg = izb.Weight(qt, wg[e0 * F:e1 * F], F, E, n_mats=n)
        Wu = izb.Weight(qt, wu[e0 * F:e1 * F], F, E, n_mats=n)
        Wd = izb.Weight(qt, wd[e0 * E:e1 * E], E, F, n_mats=n)
        offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, TM, expert_range=(e0, e1))
        ro, rt, rstok, rswt, rinv = O.moe_sort_range(ids.cpu().numpy(), wts.cpu().numpy(), counts.cpu().numpy(), TM, e0, e1)
        nt = int(tiles[0].item())
        ns = int(ro[-1])
        assert nt == rt[0] and (tiles.cpu().numpy()[:1 + 3 * nt] == rt[:1 + 3 * nt]).all()
        assert (offs.cpu().numpy() == ro).all() and (inv.cpu().numpy() == rinv).all()
        assert (stok.cpu().numpy()[:ns] == rstok[:ns]).all()
        h = izb.moe_gateup(Wg, Wu, aq, asc, tiles, max_tiles, TM, stok, Sn)
        hq, hsc, _ = izb.quantize_act(h, Mp=Sp)
        y = izb.moe_down(Wd, hq, hsc, tiles, max_tiles, TM, swt, Sn)
        part = torch.full((T, E), float("nan"), dtype=torch.float32, device="cuda")
        izb.moe_combine(part, y, inv, NU, sh=dev(torch, sh) if shared else None, sgate=sgate if shared else None, partial=True)
        ref = O.moe_combine_ex(np.zeros((T, E), np.float32), np.nan_to_num(y.cpu().numpy()), rinv, NU, sh=sh if shared else None,
                               sgate=sgate.cpu().numpy() if shared else None, partial=True)
        got = part.cpu().numpy()
        assert (bits(got) == bits(ref)).all()
        for W in (Wg, Wu, Wd):
            W.close()
        return got

    whole = dev(torch, x).clone()
    offs, tiles, max_tiles, stok, swt, inv = izb.moe_sort(ids, wts, counts, TM)
    Wg, Wu, Wd = izb.Weight(qt, wg, F, E, n_mats=NE), izb.Weight(qt, wu, F, E, n_mats=NE), izb.Weight(qt, wd, E, F, n_mats=NE)
    h = izb.moe_gateup(Wg, Wu, aq, asc, tiles, max_tiles, TM, stok, Sn)
    hq, hsc, _ = izb.quantize_act(h, Mp=Sp)
    y = izb.moe_down(Wd, hq, hsc, tiles, max_tiles, TM, swt, Sn)
    izb.moe_combine(whole, y, inv, NU, sh=dev(torch, sh), sgate=sgate)
    parts = np.stack([run(0, 3, True), run(3, NE, False)])  # (an uneven split; the shared expert on the first rank only)
    split = O.tp_add(x, parts)
    w = whole.cpu().numpy()
    assert np.abs(split - w).max() <= 2e-6 * np.abs(w).max()
    assert izb.device_status(0) == 0
    for W in (Wg, Wu, Wd):
        W.close()
