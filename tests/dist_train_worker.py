"""Worker of the two-rank data-parallel training test (launched by torchrun, one process per GPU).

Each rank trains one full-batch step on its own 256 rows; the library all-reduces the flat
gradient with NCCL.  Rank 0 then checks the summed gradient against the oracle's gradient of the
concatenated 512-row batch and that both replicas hold identical weights."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import torch
    import torch.distributed as dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    import spingalett_b200 as spg
    from oracle import OracleNet
    lib = spg.lib()
    lib.spingalett_set_verbose(False)
    assert lib.spingalett_set_device(local) == 0
    uid = np.zeros(128, np.uint8)
    if rank == 0:
        assert lib.spingalett_dist_unique_id(uid.ctypes.data) == 0
    t = torch.from_numpy(uid)
    dist.broadcast(t, 0)
    assert lib.spingalett_dist_init(rank, world, t.numpy().ctypes.data) == 0
    assert lib.spingalett_dist_world() == world

    topo, acts = [784, 512, 1000, 10], [spg.abi.ACT_RELU, spg.abi.ACT_RELU, spg.abi.ACT_SOFTMAX]
    net = spg.Network.build(topo, acts, spg.abi.WEIGHT_INITIALIZATION_HE, seed=1234)      # same seed: same replica
    onet = OracleNet.from_arrays(net.topology, net.acts, net.weights, net.biases)
    rng = np.random.default_rng(7)
    x = rng.random((256 * world, 784), dtype=np.float32)
    tg = np.zeros((256 * world, 10), np.float32)
    tg[np.arange(256 * world), rng.integers(0, 10, 256 * world)] = 1.0
    mine = slice(256 * rank, 256 * (rank + 1))
    net.train(x[mine], tg[mine], epochs=1, strategy=spg.abi.STRATEGY_FULL_BATCH, learning_rate=1e-3)
    c = net.c
    g = np.concatenate([np.ctypeslib.as_array(c.grad_weights, shape=(c.total_weights,)),
                        np.ctypeslib.as_array(c.grad_biases, shape=(c.total_biases,))]).copy()
    w = np.concatenate([net.weights, net.biases]).copy()
    gathered = [torch.zeros(w.size) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(w))
    if rank == 0:
        for other in gathered[1:]:
            assert np.array_equal(other.numpy(), w), "replicas diverged"
        # summed per-rank gradients (each scaled 1/256) = world * gradient of the whole batch scaled 1/(256*world)
        og = onet.gradients(x, tg, 1.0 / (256 * world)) * world
        rel = np.linalg.norm(g - og) / np.linalg.norm(og)
        assert rel <= 1e-4, rel
        print("DIST_TRAIN_OK rel", rel, flush=True)
    lib.spingalett_dist_shutdown()
    net.free()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
