"""Two CPU ranks under gloo: sequences are partitioned, each rank owns its
sequences' pages under local ids and computes its rows with no collective; the
verification gather on rank 0 reproduces the single-process result."""

from __future__ import annotations

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import REPO_ROOT, make_paged_inputs


def _free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _worker(rank, world, port, policy, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, str(REPO_ROOT))
    sys.path.insert(0, str(REPO_ROOT / "tests"))
    import __graft_entry__ as entry

    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        package, oracle = entry.load_package(), entry.load_oracle()
        lengths = [0, 1, 15, 16, 17, 33, 81, 100, 300]
        q, k, v, table, lens = make_paged_inputs(lengths, seed=12, poison=True)
        shards = package.sharding.partition_sequences(lengths, world, policy)
        mine = torch.tensor(shards[rank], dtype=torch.long)
        local_table, pages = package.sharding.localize_block_table(table[mine], lens[mine])
        # the rank's own pools hold only its pages, under local ids
        out = oracle.paged_attention(q[mine], k[pages], v[pages], local_table, lens[mine])
        full = package.sharding.gather_rows(out, shards[rank], len(lengths))
        if rank == 0:
            expected = oracle.paged_attention(q, k, v, table, lens)
            queue.put(bool(torch.equal(full, expected)))
        else:
            assert full is None
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("policy", ["snake", "block"])
def test_two_ranks_reproduce_the_global_result(policy):
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_worker, args=(rank, 2, port, policy, queue)) for rank in range(2)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(timeout=180)
    assert all(worker.exitcode == 0 for worker in workers), [w.exitcode for w in workers]
    assert queue.get(timeout=5) is True


def test_localize_rejects_shared_pages():
    sys.path.insert(0, str(REPO_ROOT))
    import __graft_entry__ as entry

    sharding = entry.load_package().sharding
    table = torch.tensor([[3, 4], [4, 5]], dtype=torch.int32)
    with pytest.raises(ValueError, match="shared"):
        sharding.localize_block_table(table, torch.tensor([32, 32]))
    local, pages = sharding.localize_block_table(table, torch.tensor([32, 0]))
    assert local.tolist() == [[0, 1], [0, 0]] and pages.tolist() == [3, 4]
