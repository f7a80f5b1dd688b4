"""solid_gpu_peer_sum_float: the exchange of per-GPU pairs through peer memory.

On one GPU the kernel of ONE rank runs against slots that the test fills the way the peers' stores would (two kernels
that wait on one another are never launched on one GPU); the wait that runs out is tested with a slot nobody fills and
a limit of a few milliseconds: the kernel reports it in its status word and the context stays usable.  With two or
more GPUs a second test runs real ranks as child processes (torch.distributed.run, NCCL for the set-up and the
comparison) and checks every exchange against an all-reduce of the same pairs."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _slots(world, sets=2):
    return np.zeros(sets * world * 4, dtype=np.float32)


def _put(buf, world, seq, rank, pair):
    """What rank `rank` stores into a peer's buffer for exchange number `seq`."""
    base = ((seq & 1) * world + rank) * 4
    buf[base:base + 2] = pair
    buf[base + 2:base + 3].view(np.uint32)[0] = seq


def test_pairs_are_added_in_rank_order_and_the_root_taken(gpu):
    import torch
    dev = util.Device()
    rng = np.random.default_rng(11)
    for world, rank in ((1, 0), (2, 1), (4, 0), (8, 5), (16, 15)):
        assert gpu.peer_sum_buffer_size(world) == 2 * world * 16
        for seq in (1, 2, 3):
            pairs = rng.uniform(0.5, 2.0, (world, 2)).astype(np.float32)
            host = _slots(world)
            for r in range(world):
                if r != rank:
                    _put(host, world, seq, r, pairs[r])           # the peers have delivered
            mine = dev.upload(host.view(np.uint8))
            others = [dev.upload(_slots(world).view(np.uint8)) for _ in range(world)]   # stand-ins for the peers' buffers
            buffers = [others[r].data_ptr() if r != rank else mine.data_ptr() for r in range(world)]
            local = torch.from_numpy(pairs[rank].copy()).cuda()
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            gpu.peer_sum_float(world, rank, buffers, seq, 2, local.data_ptr(), local.data_ptr(), 2, 0, status.data_ptr(), dev.stream)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            s0 = np.float32(0); s1 = np.float32(0)
            for r in range(world):
                s0 = np.float32(s0 + pairs[r, 0]); s1 = np.float32(s1 + pairs[r, 1])
            got = local.cpu().numpy()
            assert got[0] == s0 and got[1] == np.sqrt(s1), (world, rank, seq, got, s0, np.sqrt(s1))
            # what this rank stored for every peer: its pair and the sequence number, in the slot of its rank
            for r in range(world):
                seen = (others[r] if r != rank else mine).cpu().numpy().view(np.float32)
                base = ((seq & 1) * world + rank) * 4
                assert np.array_equal(seen[base:base + 2], pairs[rank]) and seen[base + 2:base + 3].view(np.uint32)[0] == seq


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(gpu):
    import torch
    dev = util.Device()
    world, rank = 2, 0
    mine, other = dev.upload(_slots(world).view(np.uint8)), dev.upload(_slots(world).view(np.uint8))
    local = torch.tensor([1.0, 4.0], dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # nobody fills slot 1: the kernel gives up after 3 ms
    gpu.peer_sum_float(world, rank, [mine.data_ptr(), other.data_ptr()], 1, 2, local.data_ptr(), local.data_ptr(), 0, 3000,
                       status.data_ptr(), dev.stream)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    # the context still works: a one-GPU exchange right after
    status.zero_()
    one = dev.upload(_slots(1).view(np.uint8))
    local = torch.tensor([3.0, 16.0], dtype=torch.float32, device="cuda")
    gpu.peer_sum_float(1, 0, [one.data_ptr()], 1, 2, local.data_ptr(), local.data_ptr(), 2, 0, status.data_ptr(), dev.stream)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and local.cpu().tolist() == [3.0, 4.0]


def test_arguments_are_checked(gpu):
    import torch
    dev = util.Device()
    buf = dev.upload(_slots(2).view(np.uint8))
    local = torch.zeros(2, dtype=torch.float32, device="cuda")
    for args in ((0, 0, [], 1, 2), (2, 2, [buf.data_ptr()] * 2, 1, 2), (2, 0, [buf.data_ptr()] * 2, 0, 2),
                 (2, 0, [buf.data_ptr()] * 2, 1, 3), (2, 0, [buf.data_ptr(), 0], 1, 2), (17, 0, [buf.data_ptr()] * 17, 1, 2)):
        world, rank, buffers, seq, count = args
        with pytest.raises(RuntimeError):
            gpu.peer_sum_float(world, rank, buffers, seq, count, local.data_ptr(), local.data_ptr(), 0, 0, 0, dev.stream)


WORKER = r'''
import os, sys
sys.path[:0] = [%(root)r, %(pkg)r]
import torch, torch.distributed as dist
from solid_b200 import shard
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
peer = shard.PeerSum.create(dev)
if peer is None:
    if rank == 0: print("PEER-UNAVAILABLE")
    dist.destroy_process_group(); sys.exit(0)
gen = torch.Generator(device="cpu"); gen.manual_seed(1234 + rank)
bad = 0
for step in range(40):
    pair = (torch.rand(2, generator=gen) + 0.5).to(dev)
    want = pair.clone(); dist.all_reduce(want)                   # NCCL adds in its own order: compare with a tolerance
    want[1] = torch.sqrt(want[1])
    got = peer.sum_pair(pair.clone(), sqrt_second=True)
    every = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(every, got)
    torch.cuda.synchronize()
    if not torch.allclose(got, want, rtol=1e-6, atol=0): bad += 1
    if any(not torch.equal(every[0], e) for e in every): bad += 1      # the same bits on every rank
peer.check()
flag = torch.tensor([bad], device=dev); dist.all_reduce(flag)
if rank == 0: print("PEER-OK" if int(flag.item()) == 0 else "PEER-MISMATCH %%d" %% int(flag.item()))
dist.destroy_process_group()
'''


def test_real_ranks_agree_with_the_all_reduce(tmp_path):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 4 if n >= 4 else 2
    script = tmp_path / "peer_worker.py"
    script.write_text(WORKER % {"root": str(ROOT), "pkg": str(ROOT / "ocean-tensor-package_b200")})
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:]
    if "PEER-UNAVAILABLE" in res.stdout:
        pytest.skip("symmetric memory cannot be set up on this machine")
    assert "PEER-OK" in res.stdout, res.stdout[-3000:]
