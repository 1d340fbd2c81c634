"""The expert-parallel scheme on CPU: two gloo ranks as child processes."""
import os
import socket
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def test_local_picks_partition(pkg):
    host = pkg.host
    rng = np.random.default_rng(0)
    E, K, G, tl = 64, 6, 4, 2
    T = G * tl
    ids = np.stack([rng.choice(E, K, replace=False) for _ in range(T)]).astype(np.int32)
    wts = rng.random((T, K)).astype(np.float32)
    seen = np.zeros((T, K), int)
    shared = np.zeros(T, int)
    for r in range(G):
        first, count = host.ep_expert_range(r, G, E)
        lids, lw = host.ep_local_picks(ids, wts, r, G, E, tl, True)
        m = lids[:, :K] >= 0
        assert ((ids[m] - first) == lids[:, :K][m]).all() and (lids[:, :K][m] < count).all()
        assert (lw[:, :K][m] == wts[m]).all() and (lw[:, :K][~m] == 0).all()
        seen += m
        shared += lids[:, K] == count
    assert (seen == 1).all() and (shared == 1).all()


def test_two_rank_layer_matches_single_process():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "ep_worker.py")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o[-2000:]
        assert "rank %d ok" % r in o
