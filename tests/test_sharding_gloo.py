"""Multi-rank host logic on CPU: 2 gloo ranks shard a graph by destination ranges, all-gather the
source features and each evaluate their rows with the oracle; the union must equal the 1-rank result."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from e3nn_b200 import sharding
from oracle import e3nn_oracle as orc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _graph():
    torch.manual_seed(0)
    N = 37
    deg = torch.randint(0, 7, (N,))
    deg[3] = 0
    deg[20] = 25
    dst = torch.repeat_interleave(torch.arange(N), deg)
    E = dst.numel()
    rowptr = torch.zeros(N + 1, dtype=torch.int64)
    rowptr[1:] = torch.cumsum(deg, 0)
    mid, ins = orc.conv_uvu_layout("4x0e+4x1o", "0e+1o+2e", [(0, 1), (1, -1), (1, 1), (2, 1)])
    wn = sum(m for m, _, _ in orc.parse_irreps(mid))
    return dict(N=N, E=E, dst=dst, rowptr=rowptr, src=torch.randint(0, N, (E,)), x=torch.randn(N, 16).double(),
                vec=torch.randn(E, 3).double(), w=torch.randn(E, wn).double(), mid=mid, ins=ins)


def _conv(g, x, src, dst, vec, w, n):
    return orc.conv_uvu("4x0e+4x1o", "0e+1o+2e", g["mid"], g["ins"], x, vec, src, dst, w, n, [0, 1, 2])


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = _graph()
    bounds = sharding.partition_rows_by_edges(g["rowptr"], world)
    n0, n1, e0, e1, rp = sharding.local_shard(g["rowptr"], bounds, rank)
    x_full = sharding.all_gather_rows(g["x"][n0:n1].clone(), bounds)   # each rank owns only its rows
    assert torch.equal(x_full, g["x"])
    # asynchronous form: work may be enqueued between the call and wait(); the result is complete after wait()
    out = torch.full_like(g["x"], float("nan"))
    same, wait = sharding.all_gather_rows(g["x"][n0:n1].clone(), bounds, out=out, async_op=True)
    assert same is out
    wait()
    assert torch.equal(out, g["x"])
    local = _conv(g, x_full, g["src"][e0:e1], g["dst"][e0:e1] - n0, g["vec"][e0:e1], g["w"][e0:e1], n1 - n0)
    torch.save((bounds, n0, n1, e0, e1, rp, local), os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = _graph()
    full = _conv(g, g["x"], g["src"], g["dst"], g["vec"], g["w"], g["N"])
    parts = [torch.load(os.path.join(tmp_path, f"r{r}.pt")) for r in range(world)]
    bounds = parts[0][0]
    assert bounds[0] == 0 and bounds[-1] == g["N"] and bounds == sorted(bounds)
    edges = 0
    for r, (b, n0, n1, e0, e1, rp, local) in enumerate(parts):
        assert b == bounds and (n0, n1) == (bounds[r], bounds[r + 1])
        assert int(rp[0]) == 0 and int(rp[-1]) == e1 - e0 and rp.numel() == n1 - n0 + 1
        assert torch.allclose(local, full[n0:n1], rtol=0, atol=1e-12)
        edges += e1 - e0
    assert edges == g["E"]
    # balance: no part holds more than its share plus the longest row
    share = g["E"] / world
    assert all(abs((p[4] - p[3]) - share) <= 25 for p in parts)


def test_partition_edge_cases():
    rowptr = torch.tensor([0, 0, 0, 5, 5, 9])
    for world in (1, 2, 3, 8):
        b = sharding.partition_rows_by_edges(rowptr, world)
        assert len(b) == world + 1 and b[0] == 0 and b[-1] == 5 and b == sorted(b)
    assert sharding.partition_rows_by_edges(torch.tensor([0]), 4) == [0, 0, 0, 0, 0]


def test_partition_prefers_equal_rows_when_edges_balance():
    # uniform degrees: equal row counts (one all_gather_into_tensor instead of a group of unequal broadcasts)
    deg = torch.full((64,), 10)
    deg[::7] += 1                                   # within 1 % of balance per part
    rowptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(deg, 0)])
    assert sharding.partition_rows_by_edges(rowptr, 4) == [0, 16, 32, 48, 64]
    # a skewed graph keeps the split by edges
    deg = torch.ones(64, dtype=torch.int64)
    deg[:8] = 100
    rowptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(deg, 0)])
    b = sharding.partition_rows_by_edges(rowptr, 4)
    assert b != [0, 16, 32, 48, 64] and b[0] == 0 and b[-1] == 64 and b == sorted(b)
    parts = [int(rowptr[b[r + 1]] - rowptr[b[r]]) for r in range(4)]
    assert max(parts) <= 2 * int(rowptr[-1]) // 4


def _timeout_worker(rank, world, port, out_dir):
    """Rank 1 leaves between steps (it never joins the second collective); rank 0's collective must end with an
    error after the process-group timeout instead of waiting for ever."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sharding.init_process_group("gloo", timeout_s=3.0)
    x = torch.ones(4) * (rank + 1)
    dist.all_reduce(x)                     # step 1: both ranks
    assert float(x[0]) == 3.0
    if rank == 1:
        torch.save("left", os.path.join(out_dir, "r1.pt"))
        os._exit(0)                        # leaves with nothing in flight
    try:
        dist.all_reduce(x)                 # step 2: the peer is gone
        outcome = "no error"
    except Exception as exc:               # gloo: a RuntimeError naming the timeout or the closed connection
        outcome = f"error: {type(exc).__name__}"
    torch.save(outcome, os.path.join(out_dir, "r0.pt"))
    os._exit(0)


def test_collective_with_a_missing_rank_times_out(tmp_path):
    world = 2
    mp.spawn(_timeout_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert torch.load(os.path.join(tmp_path, "r1.pt")) == "left"
    assert torch.load(os.path.join(tmp_path, "r0.pt")).startswith("error")
