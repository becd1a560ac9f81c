"""The N>1 host path on CPU: two gloo ranks each own a column shard of an NVFP4 LM head, produce
their (max, index) keys with the oracle standing in for the GPU kernel, all-gather the keys the
way ShardedLmHead does and fold them; the result must equal the unsharded argmax."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from oracle import cpu as C
    from qwen38_flash_ops_b200 import lmhead_shard as LS
    from qwen38_flash_ops_b200 import packing as P

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(1234)                      # same data on every rank
    K, N, M = 128, 128 * 5, 4
    w = P.synth_weight(rng, K, N)
    w[:, 130] = w[:, 500]                                  # equal columns in different shards: a cross-shard tie
    pk = P.pack_nvfp4(w)
    pk = P.pack_nvfp4(O_dequant(pk, N))                    # re-pack so both columns share bytes exactly
    x = P.synth_x(rng, M, K)
    c0, c1 = LS.ShardedLmHead.column_range(N, rank, world)
    shard = P.nvfp4_column_slice(pk, N, c0, c1)
    logits, _, _ = C.skinny_gemm(2, x, shard, c1 - c0, None)
    idx, val = C.argmax_rows(0, logits)
    key = torch.from_numpy(LS.pack_key(val, idx + c0).view(np.int64))
    gathered = torch.empty(world * M, dtype=torch.int64)
    dist.all_gather_into_tensor(gathered, key)
    gi, gv = LS.fold_keys_host(gathered.numpy().reshape(world, M))
    full, _, _ = C.skinny_gemm(2, x, pk, N, None)
    ei, ev = C.argmax_rows(0, full)
    np.save(os.path.join(out_dir, f"r{rank}.npy"), np.stack([gi, ei, gv.view(np.int32), ev.view(np.int32)]))
    dist.barrier()
    dist.destroy_process_group()


def O_dequant(pk, n):
    from oracle import oracle as O

    return O.decode_weights_exact(2, pk, n)


@pytest.mark.parametrize("world", [2])
def test_two_rank_sharded_lmhead_on_gloo(tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    res = [np.load(tmp_path / f"r{r}.npy") for r in range(world)]
    for r in res:
        assert np.array_equal(r[0], r[1]), "sharded argmax differs from the unsharded one"
        assert np.array_equal(r[2], r[3])
    assert np.array_equal(res[0], res[1]), "ranks disagree"
