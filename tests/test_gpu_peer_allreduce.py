"""The peer-memory sum of K-sharded partial results (gsq_allreduce_sum, gsq_b200.tp.PeerAllReduce).

  * on one GPU: two "ranks" whose buffers and flag pads all live on this GPU (the kernel only sees pointers): the sum,
    its rank order, the epoch counter over several calls -- and a wait that runs out: a call for which the other
    rank's flag is never set returns after its bounded wait, raises gsq_allreduce_error_flag, leaves the context
    usable, and the next well-formed call is correct;
  * on 2+ GPUs (skipped otherwise): child processes, one per GPU, over torch's symmetric memory, eager and inside
    a CUDA graph, against a host-formed sum."""

import ctypes
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


def _ptrs(ts):
    return torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=DEV)


def test_two_ranks_emulated_on_one_gpu_and_a_wait_that_runs_out():
    from gsq_b200 import _cabi

    lib = _cabi.lib
    n = 4096
    parts = [torch.randn(n, device=DEV).to(torch.bfloat16) for _ in range(2)]
    pads = [torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(2)]
    state = [torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(2)]
    outs = [torch.zeros(n, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    bufs, flags = _ptrs(parts), _ptrs(pads)
    st = torch.cuda.current_stream().cuda_stream

    def call(rank):
        return lib.gsq_allreduce_sum(bufs.data_ptr(), flags.data_ptr(), rank, 2, n, 2, outs[rank].data_ptr(),
                                     state[rank].data_ptr(), st)
    flag = ctypes.c_int(-1)
    assert lib.gsq_allreduce_error_flag(ctypes.byref(flag)) == 0
    before = flag.value
    # rank 0 alone: rank 1 never signals epoch 1, so rank 0's wait runs out (bounded), nothing is written
    assert call(0) == 0
    torch.cuda.synchronize()
    assert lib.gsq_allreduce_error_flag(ctypes.byref(flag)) == 0 and flag.value == 1
    assert not outs[0].any()
    assert before in (0, 1)
    # the context is still usable. Rank 1 now makes its first call: it finds rank 0's flag of epoch 1 and completes.
    assert call(1) == 0
    torch.cuda.synchronize()
    want = (parts[0].float() + parts[1].float()).to(torch.bfloat16)
    assert torch.equal(outs[1], want)
    # second epoch, done properly: the kernels of two ranks on one GPU must not wait on each other, so each flag is
    # set by hand before the other rank's call (what the peer's kernel would have stored)
    pads[0][1] = 2      # "rank 1 has finished its partial of epoch 2"
    assert call(0) == 0
    torch.cuda.synchronize()
    assert torch.equal(outs[0], want)
    assert call(1) == 0  # rank 0's kernel above stored its flag of epoch 2 into rank 1's pad
    torch.cuda.synchronize()
    assert torch.equal(outs[1], want)
    assert int(state[0][0]) == 2 and int(state[1][0]) == 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ranks_on_separate_gpus():
    n = min(4, torch.cuda.device_count())
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29533",
                        os.path.join(ROOT, "tests", "_peer_allreduce_worker.py")], capture_output=True, text=True,
                       timeout=300, env=env)
    assert p.returncode == 0 and "peer all-reduce ok" in p.stdout, (p.stdout[-1500:], p.stderr[-3000:])
    print(p.stdout.strip().splitlines()[-1])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_product_fused_with_its_sum():
    """gsq_linear_allreduce: the K-sharded product and the sum of its result over the GPUs in one kernel per rank,
    bit for bit against product + gathered sum in rank order, eagerly and in a CUDA graph."""
    n = min(4, torch.cuda.device_count())
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29535",
                        os.path.join(ROOT, "tests", "_fused_allreduce_worker.py")], capture_output=True, text=True,
                       timeout=400, env=env)
    assert p.returncode == 0 and "fused product + sum ok" in p.stdout, (p.stdout[-1500:], p.stderr[-3000:])
    print(p.stdout.strip().splitlines()[-1])
