"""One rank of the CPU model of the expert-parallel layer (gloo, world size 2).

The expert arithmetic is the CPU oracle; what is under test is the partition and the
exchange: ranks gather rows and picks, each computes only its own experts (plus the
shared expert for its own tokens), partial rows go back to the owners and are summed
in rank order.  The result must equal the single-process layer."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402
from oracle import pyoracle  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%s" % os.environ["MASTER_PORT"],
                            rank=rank, world_size=world)
    pkg = entry.load_package()
    host = pkg.host
    O = pyoracle.oracle()
    H, F, E, K, t_local = 512, 256, 16, 4, 3
    T = world * t_local
    L = pkg.synth.layer(7, E, H, F)
    xs = pkg.synth.hidden(8, T, H)
    first, count = host.ep_expert_range(rank, world, E)
    # 1. own tokens: norm, router, top-k
    own = slice(rank * t_local, (rank + 1) * t_local)
    xn_l = np.stack([O.rms_norm(x, L["norm_w"], 1e-6) for x in xs[own]])
    picks = [O.topk(O.softmax(O.gemv_f32(L["router"], x)), K, True) for x in xn_l]
    ids_l = np.stack([p[0] for p in picks]).astype(np.int32)
    wts_l = np.stack([p[1] for p in picks]).astype(np.float32)
    # 2. dispatch: gather rows and picks
    def gather(a):
        out = [torch.empty_like(torch.from_numpy(a)) for _ in range(world)]
        dist.all_gather(out, torch.from_numpy(np.ascontiguousarray(a)))
        return np.concatenate([o.numpy() for o in out])
    xn, ids, wts = gather(xn_l), gather(ids_l), gather(wts_l)
    # 3. local experts
    lids, lw = host.ep_local_picks(ids, wts, rank, world, E, t_local, True)
    local_packs = [L["experts"][first + j] for j in range(count)] + [L["shared"]]
    partial = np.zeros((T, H), np.float32)
    for t in range(T):
        sel = [k for k in range(K + 1) if lids[t, k] >= 0]
        if sel:
            partial[t] = O.expert_job([local_packs[lids[t, k]] for k in sel], lw[t, sel], xn[t], H, F)
    # 4. combine: every rank sends the rows of rank p's tokens to p
    recv = [torch.empty(t_local, H) for _ in range(world)]
    send = [torch.from_numpy(np.ascontiguousarray(partial[p * t_local:(p + 1) * t_local])) for p in range(world)]
    reqs = []
    for p in range(world):
        if p == rank:
            recv[p].copy_(send[p])
        else:
            reqs.append(dist.isend(send[p], p))
            reqs.append(dist.irecv(recv[p], p))
    for r in reqs:
        r.wait()
    y = np.zeros((t_local, H), np.float32)
    for s in range(world):
        y = y + recv[s].numpy()
    # check against the single-process layer
    worst = 0.0
    for i, t in enumerate(range(rank * t_local, (rank + 1) * t_local)):
        y0, ids0, _, _ = O.moe_layer(xs[t], L["norm_w"], 1e-6, L["router"], K, L["experts"], L["shared"], H, F)
        assert ids0.tolist() == ids[t].tolist()
        worst = max(worst, float(np.linalg.norm(y[i] - y0) / np.linalg.norm(y0)))
    assert worst < 1e-5, worst
    # The one-collective form: every rank norms and routes ALL tokens, computes its own experts
    # (the shared expert for its own tokens) and one all-reduce sums the partial rows everywhere.
    xn_a = np.stack([O.rms_norm(x, L["norm_w"], 1e-6) for x in xs])
    picks_a = [O.topk(O.softmax(O.gemv_f32(L["router"], x)), K, True) for x in xn_a]
    ids_a = np.stack([p[0] for p in picks_a]).astype(np.int32)
    wts_a = np.stack([p[1] for p in picks_a]).astype(np.float32)
    assert np.array_equal(ids_a, ids) and np.array_equal(wts_a, wts)      # replicated routing = gathered routing
    total = torch.from_numpy(partial.copy())
    dist.all_reduce(total)
    worst_ar = 0.0
    for t in range(T):
        y0 = O.moe_layer(xs[t], L["norm_w"], 1e-6, L["router"], K, L["experts"], L["shared"], H, F)[0]
        worst_ar = max(worst_ar, float(np.linalg.norm(total.numpy()[t] - y0) / np.linalg.norm(y0)))
    assert worst_ar < 1e-5, worst_ar
    # every pick is owned by exactly one rank
    owned = torch.from_numpy((lids[:, :K] >= 0).astype(np.int32))
    dist.all_reduce(owned)
    assert (owned.numpy() == 1).all()
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok %.2e" % (rank, worst))


if __name__ == "__main__":
    main()
