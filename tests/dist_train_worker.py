"""Worker of the two-rank data-parallel training test (launched by torchrun, one process per GPU).

Each rank trains on its own 256 rows, once with the one-kernel exchange over peer memory and once with the NCCL
all-reduce: the summed gradient of a full-batch step against the oracle's gradient of the concatenated batch, and
weights, gradients and optimiser moments bit-identical on every rank after full-batch and mini-batch steps."""
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
    rng = np.random.default_rng(7)
    x = rng.random((256 * world, 784), dtype=np.float32)
    tg = np.zeros((256 * world, 10), np.float32)
    tg[np.arange(256 * world), rng.integers(0, 10, 256 * world)] = 1.0
    mine = slice(256 * rank, 256 * (rank + 1))

    def flat(c, a, b, na, nb):
        return np.concatenate([np.ctypeslib.as_array(getattr(c, a), shape=(na,)), np.ctypeslib.as_array(getattr(c, b), shape=(nb,))]).copy()

    def same_everywhere(v, what):
        gathered = [torch.zeros(v.size) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(v))
        for other in gathered:
            assert np.array_equal(other.numpy(), v), what + ": replicas diverged"

    results = {}
    # the one-kernel exchange over peer memory (default) and the NCCL all-reduce
    for mode in ("p2p", "nccl"):
        os.environ["SPINGALETT_EXCHANGE"] = mode
        net = spg.Network.build(topo, acts, spg.abi.WEIGHT_INITIALIZATION_HE, seed=1234)      # same seed: same replica
        onet = OracleNet.from_arrays(net.topology, net.acts, net.weights, net.biases)
        # one full-batch step: the summed gradient against the oracle's gradient of the concatenated batch
        net.train(x[mine], tg[mine], epochs=1, strategy=spg.abi.STRATEGY_FULL_BATCH, learning_rate=1e-3)
        c = net.c
        nw, nb = int(c.total_weights), int(c.total_biases)
        g = flat(c, "grad_weights", "grad_biases", nw, nb)
        w = np.concatenate([net.weights, net.biases]).copy()
        same_everywhere(w, mode + " weights")
        same_everywhere(g, mode + " summed gradients")
        # summed per-rank gradients (each scaled 1/256) = world * gradient of the whole batch scaled 1/(256*world)
        og = onet.gradients(x, tg, 1.0 / (256 * world)) * world
        rel = np.linalg.norm(g - og) / np.linalg.norm(og)
        assert rel <= 1e-4, (mode, rel)
        # several mini-batch steps with decay (AdamW): weights and both moments identical on every rank afterwards
        net.train(x[mine], tg[mine], epochs=3, batch_size=64, learning_rate=1e-3, optimizer=spg.abi.OPTIMIZER_ADAMW, weight_decay=1e-2)
        w2 = np.concatenate([net.weights, net.biases]).copy()
        m2 = flat(net.c, "opt_m_weights", "opt_m_biases", nw, nb)
        v2 = flat(net.c, "opt_v_weights", "opt_v_biases", nw, nb)
        same_everywhere(w2, mode + " weights after mini-batch steps")
        same_everywhere(m2, mode + " first moments")
        same_everywhere(v2, mode + " second moments")
        assert np.all(np.isfinite(w2)) and np.any(m2 != 0) and np.any(v2 != 0) and not np.array_equal(w2, w)
        results[mode] = (g, w, w2, m2, v2)
        net.free()
    # the two exchanges add the ranks' gradients in different orders: the summed gradients agree to fp32 rounding of the
    # sums; weights and moments after Adam steps agree loosely (an element whose gradient is rounding noise may step the
    # other way), which is a sanity check, not a parity claim -- the claims are the per-mode checks above
    names = ("summed gradient", "weights after one step", "weights after mini-batch steps", "first moments", "second moments")
    for name, a_, b_ in zip(names, results["p2p"], results["nccl"]):
        diff = float(np.abs(a_ - b_).max())
        bound = (1e-5 if name == "summed gradient" else 5e-3) * max(1.0, float(np.abs(b_).max()))
        assert diff <= bound, (name, diff, bound)
    if rank == 0:
        print("DIST_TRAIN_OK rel", rel, flush=True)
    lib.spingalett_dist_shutdown()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        # torchrun's own summary buries the rank's traceback: leave it where the test can find it
        import traceback
        with open(os.path.join(sys.argv[1], f"rank{os.environ.get('RANK', '0')}.err"), "w") as f:
            traceback.print_exc(file=f)
        raise
