"""World-size-2 gloo runs (CPU) of the multi-GPU host logic: token sharding + all-reduce of dW,
and row sharding with the global-gamma exchange.  The per-rank arithmetic is done by the CPU
oracle here; on GPUs the same module drives the CUDA kernels (bench.py --gpus N)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import normal_f32


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from alice_train import parallel
        from oracle import pyoracle as orc
        m, out, inn = 24, 12, 20
        w_lat = normal_f32(1, (out, inn), 0.02)
        x, dy = normal_f32(2, (m, inn)), normal_f32(3, (m, out), 1e-2)
        g, codes, _ = orc.quantize_and_pack(w_lat)
        wq = codes.reshape(out, inn).astype(np.float32) * np.float32(g)

        # --- data parallel over tokens: dW is the only exchange
        t0, t1 = parallel.token_shard(m, world, rank)
        _, dw_local = orc.matmul_bt_backward(dy[t0:t1], x[t0:t1], wq, t1 - t0, out, inn, want=("db",))
        dw = torch.from_numpy(dw_local.copy())
        red = parallel.DwAllReducer()
        red.submit(dw)
        red.wait()
        _, dw_full = orc.matmul_bt_backward(dy, x, wq, m, out, inn, want=("db",))
        e_dw = float(np.max(np.abs(dw.numpy() - dw_full)) / np.max(np.abs(dw_full)))

        # --- row shards: global gamma from 8-byte partial sums, forward gather, dx reduce
        r0, r1 = parallel.row_shard(out, world, rank)
        shard = w_lat[r0:r1]
        s_local = torch.tensor([float(np.sum(np.abs(shard).astype(np.float64)))], dtype=torch.float64)
        gamma = parallel.global_gamma(s_local, out * inn)
        same_gamma = float(gamma.item()) == g
        inv = np.float32(1.0) / np.float32(gamma.item())
        codes_shard = np.clip(np.round(shard * inv), -1, 1)  # no ties in this draw; full rule is in the oracle
        same_codes = bool(np.array_equal(codes_shard.astype(np.int8), codes.reshape(out, inn)[r0:r1]))
        xq, s = orc.act_quant_int8(x)
        acc_local = orc.int8_ternary_acc(xq, codes.reshape(out, inn)[r0:r1].copy())
        acc = parallel.gather_rows(torch.from_numpy(acc_local))
        same_acc = bool(np.array_equal(acc.numpy(), orc.int8_ternary_acc(xq, codes.reshape(out, inn))))
        dx_part, _ = orc.matmul_bt_backward(np.ascontiguousarray(dy[:, r0:r1]), x, wq[r0:r1].copy(), m, r1 - r0, inn,
                                            want=("da",))
        dx = parallel.reduce_dx(torch.from_numpy(dx_part.copy()))
        dx_full, _ = orc.matmul_bt_backward(dy, x, wq, m, out, inn, want=("da",))
        e_dx = float(np.max(np.abs(dx.numpy() - dx_full)) / np.max(np.abs(dx_full)))
        q.put((rank, e_dw, same_gamma, same_codes, same_acc, e_dx))
    finally:
        dist.destroy_process_group()


def test_dp_and_rowshard_world2():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, e_dw, same_gamma, same_codes, same_acc, e_dx in res:
        assert e_dw <= 1e-5 and e_dx <= 1e-5, (rank, e_dw, e_dx)
        assert same_gamma and same_codes and same_acc, rank


def test_shard_arithmetic():
    from alice_train import parallel
    for n, w in [(4096, 8), (10, 3), (7, 8), (0, 2)]:
        cuts = [parallel.token_shard(n, w, r) for r in range(w)]
        assert cuts[0][0] == 0 and cuts[-1][1] == n
        assert all(cuts[i][1] == cuts[i + 1][0] for i in range(w - 1))
        assert max(b - a for a, b in cuts) - min(b - a for a, b in cuts) <= 1
    for out, w, al in [(28672, 8, 128), (1000, 4, 128), (8192, 8, 256)]:
        cuts = [parallel.row_shard(out, w, r, al) for r in range(w)]
        assert cuts[0][0] == 0 and cuts[-1][1] == out
        assert all(a % al == 0 for a, _ in cuts)
