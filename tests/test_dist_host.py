"""Host-side pieces of the multi-process paths, run as two gloo ranks on the CPU: the id exchange
used to set up the gradient communicator, row sharding of a batch across ranks, and the max-over-ranks
reduction the benchmark uses for its timing, and the argument agreement a data-parallel train() begins with."""
import os
import subprocess
import sys
import textwrap

WORKER = textwrap.dedent('''
    import os, sys
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, os.environ["SPG_ROOT"])
    import spingalett_b200 as spg
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    # 1. the 128-byte communicator id travels from rank 0 to everyone over the host channel
    uid = np.zeros(128, np.uint8)
    if rank == 0:
        uid[:] = np.random.default_rng(1).integers(0, 256, 128, dtype=np.uint8)
    t = torch.from_numpy(uid)
    dist.broadcast(t, 0)
    assert np.array_equal(t.numpy(), np.random.default_rng(1).integers(0, 256, 128, dtype=np.uint8))
    # 2. rows of a batch are cut contiguously and cover it exactly once
    lo, hi = spg.shard_rows(65537, world, rank)
    spans = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(spans, torch.tensor([lo, hi]))
    flat = [int(v) for s in spans for v in s]
    assert flat[0] == 0 and flat[-1] == 65537 and all(flat[2 * i + 1] == flat[2 * i + 2] for i in range(world - 1))
    assert max(flat[2 * i + 1] - flat[2 * i] for i in range(world)) - min(flat[2 * i + 1] - flat[2 * i] for i in range(world)) <= 1
    # 3. timing is the max over ranks
    ms = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    assert ms.item() == float(world)
    # 4. without a GPU the communicator cannot come up and the library says so instead of pretending
    if spg.lib().spingalett_get_device_count() == 0:
        assert spg.lib().spingalett_dist_init(rank, world, t.numpy().ctypes.data) != 0
        spg.lib().spingalett_clear_error()
    assert spg.lib().spingalett_dist_init(0, 1, None) == 0 and spg.lib().spingalett_dist_world() == 1
    # 5. the argument agreement a data-parallel train() starts with: equal arguments pass on every rank, a rank with a
    #    different sample count makes every rank refuse (the sum over ranks is what NCCL computes on the GPU)
    import ctypes as C
    lib, a = spg.lib(), spg.abi
    def packed(samples):
        args = a.TrainArgs()
        args.sample_count, args.batch_size, args.epochs = samples, 256, 10
        args.training_strategy, args.optimizer_type = a.STRATEGY_SMALL_BATCH, a.OPTIMIZER_ADAM
        buf = np.zeros(lib.spingalett_dist_agreement_floats(), np.float32)
        lib.spingalett_dist_pack_agreement(C.byref(args), buf.ctypes.data_as(a.f32p))
        return buf
    for samples, agree in ((5120, 1), (5120 + rank, 0)):
        mine = packed(samples)
        summed = torch.from_numpy(mine.copy())
        dist.all_reduce(summed)
        assert lib.spingalett_dist_check_agreement(summed.numpy().ctypes.data_as(a.f32p), mine.ctypes.data_as(a.f32p), world) == agree
    dist.barrier()
    dist.destroy_process_group()
    print("HOST_DIST_OK", rank)
''')


def test_two_gloo_ranks_host_logic(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, SPG_ROOT=root, CUDA_VISIBLE_DEVICES="")
    import socket
    with socket.socket() as sk:                     # a port nobody else on this machine is using right now
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("HOST_DIST_OK") == 2
