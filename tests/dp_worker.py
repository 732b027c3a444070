"""Worker launched once per rank by the data-parallel tests (not a test module itself).

    python dp_worker.py cpu  <rank> <world> <port> <out.npz>     gloo ranks on CPU: the exchange protocol with the oracle's gradients
    python dp_worker.py gpu  <rank> <world> <port> <out.npz>     one GPU per rank: the library's trainer and its gradient exchange (peer
                                                                 memory, or NCCL with TALOS_COMM_NO_P2P=1)
    python dp_worker.py gpu_stall <rank> <world> <port> <out.npz>  as gpu, but after one good step the LAST rank leaves out its publication
                                                                 once: every other rank's bounded wait must run out and report TIMEOUT
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

N, OBS, HID, ACT, MB, EPOCHS = 4096, 64, 256, 16, 1024, 2      # global problem: N transitions, global minibatch MB


def problem():
    import oracle as orc
    from gpu_util import normal, xavier
    obs = normal(30, (N, OBS)); act = orc.rng_bounded(31, N, ACT); adv = normal(32, (N,)); ret = normal(33, (N,))
    params = dict(w1=xavier(34, OBS, HID), b1=np.zeros(HID), w2=xavier(35, HID, HID), b2=np.zeros(HID), wp=xavier(36, HID, ACT), bp=np.zeros(ACT),
                  wv=xavier(37, HID, 1), bv=np.zeros(1))
    return obs, act, adv, ret, params


def main():
    kind, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    import oracle as orc
    from oracle import model as om
    obs, act, adv, ret, params = problem()
    model = om.MlpActorCritic(params)
    old = orc.f32r(model.log_prob(obs, act))
    mb_local = MB // world
    # rank r owns the r-th slice of every global minibatch: [s + r*mb_local, s + (r+1)*mb_local)
    if kind == "cpu":
        dist.init_process_group("gloo", rank=rank, world_size=world)
        names = model.NAMES
        m = [np.zeros_like(model.p[k]) for k in names]; v = [np.zeros_like(model.p[k]) for k in names]; t = 0
        kls = []
        for _ in range(EPOCHS):
            kl_sum = cnt = 0.0
            for s in range(0, N, MB):
                lo = s + rank * mb_local; hi = lo + mb_local
                g, loss, kl = model.grads(obs[lo:hi], act[lo:hi], old[lo:hi], adv[lo:hi], ret[lo:hi], denom=1.0)     # SUMS over local samples
                flat = np.concatenate([g[k].ravel() for k in names] + [np.array([loss, kl, float(hi - lo)])])
                buf = torch.from_numpy(flat); dist.all_reduce(buf, op=dist.ReduceOp.SUM)                             # one exchange per step
                flat = buf.numpy(); count = flat[-1]; kl_sum += flat[-2]; cnt += count
                grads, o = [], 0
                for k in names:
                    n = model.p[k].size; grads.append(flat[o:o + n].reshape(model.p[k].shape) / count); o += n         # divide by the GLOBAL count
                t += 1
                om.adam_step([model.p[k] for k in names], grads, m, v, t, np.float64(np.float32(3e-4)))
            kls.append(kl_sum / cnt)
        np.savez(out, kls=np.array(kls), **model.p)
        dist.destroy_process_group()
        return
    from __graft_entry__ import load_package
    talos = load_package()
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = talos.torch_context(rank)
    comm = None
    if world > 1:
        uid = [talos.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = talos.Comm(ctx, uid[0], world, rank)
    mode = int(os.environ.get("TALOS_TEST_MODE", "1"))
    tr = talos.PPOTrainer(ctx, talos.PpoConfig(OBS, HID, ACT, mb_local, mode), comm); tr.set_params(params)
    # gather this rank's slices of every global minibatch into one contiguous local shard
    idx = np.concatenate([np.arange(s + rank * mb_local, s + (rank + 1) * mb_local) for s in range(0, N, MB)])
    dev = lambda a, dt: torch.tensor(np.ascontiguousarray(a[idx]), dtype=dt, device="cuda")
    peer = bool(comm.peer_exchange_active) if comm else False
    d = [dev(obs, torch.float32), dev(act, torch.int32), dev(old, torch.float32), dev(adv, torch.float32), dev(ret, torch.float32)]
    if kind == "gpu_stall":
        assert peer, "the stall scenario needs the peer-memory exchange"
        tr.step(*d, mb_local); before = tr.get_params()                     # one good step
        talos.lib.talos_debug_comm_stall(comm.handle, 1 if rank == world - 1 else 0, 200000)
        tr.step(*[t[mb_local:] for t in d], mb_local)
        status = 0
        try:
            tr.last_loss()
        except talos.TalosError as e:
            status = e.status
        after = tr.get_params()
        unchanged = all(np.array_equal(before[k], after[k]) for k in before)
        dist.barrier()                                                      # every rank is between steps, nothing in flight
        np.savez(out, status=status, unchanged=unchanged, peer=peer)
        tr.close(); comm.close(); dist.destroy_process_group()
        return
    kls = tr.update(*d, idx.size, EPOCHS)
    got = tr.get_params()
    np.savez(out, kls=np.array(kls), peer=peer, **{k: v.astype(np.float64) for k, v in got.items()})
    tr.close()
    if comm: comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
