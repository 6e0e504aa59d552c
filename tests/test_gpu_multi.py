"""Two NCCL ranks on two GPUs: KV-head sharding and the sequence split (row windows of one packed
layer, all-gather + log-sum-exp combine) against the unsplit single-GPU result and the oracle.
Skipped on a single-GPU box.  NVLS is switched off so that a failing rank cannot disturb its
peer; every wait has a time limit and the parent never leaves a rank behind."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    ok = False
    try:
        from oracle import ref_attention as RA
        from oracle import ref_packing as RP
        from rdkv_b200 import sharding, synth
        from rdkv_b200.decode import DecodeTable, packed_decode_attention
        from rdkv_b200.packing import pack_kv
        H_kv, g, T, N = 4, 4, 2048, 512
        dev = torch.device("cuda", rank)
        views = []
        for i in range(3):
            seed = synth.unit_seed(4, i, 0)
            K, V = synth.make_kv(H_kv, T, seed=seed)
            vb = synth.make_v_bits(H_kv, T, N, seed=seed, per_head_N=[512, 300, 448, 129] if i == 1 else None)
            kb = synth.make_k_bits(H_kv, seed=seed)
            views.append((K, V, vb, kb))
        q = synth.make_q(H_kv * g, seed=77, batch=3, dtype=torch.bfloat16)
        layers, nvs = zip(*[pack_kv(K.to(dev), V.to(dev), vb.to(dev), kb.to(dev), g) for K, V, vb, kb in views])
        # the unsplit result on this GPU, and the oracle's on the same inputs
        tb = DecodeTable(layers, nvs, H_kv * g)
        want = packed_decode_attention(q.to(dev), tb)
        oracle = np.stack([RA.decode_attention(q[i].float().numpy(), *RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g))[0]
                           for i, (K, V, vb, kb) in enumerate(views)])
        # sequence split across the two ranks: each attends over its window of every head's rows of the SAME packed layers
        sharding.check_group_consistency(tb.n_views * tb.H_q)
        got_seq = sharding.sequence_split_attention(q.to(dev), tb)
        err_seq = float((got_seq - want).abs().max())
        e = np.abs(got_seq.cpu().numpy() - oracle)
        ok_oracle = bool(np.all(e <= 2e-3 + 1e-2 * np.abs(oracle)))
        # head sharding: each rank serves half of the heads; gather and compare with all heads here
        h0, h1 = sharding.head_shard(rank, world, H_kv)
        sl, sn = zip(*[pack_kv(*[t.to(dev) for t in sharding.shard_heads(K, V, vb, kb, rank, world)], g)
                       for K, V, vb, kb in views])
        tbh = DecodeTable(sl, sn, (h1 - h0) * g)
        mine = packed_decode_attention(q.to(dev)[:, h0 * g:h1 * g].contiguous(), tbh)
        outs = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(outs, mine)
        got_heads = torch.cat(outs, dim=1)
        err_heads = float((got_heads - want).abs().max())
        tb.check_status(); tbh.check_status()
        ret[rank] = (err_seq, err_heads, ok_oracle)
        ok = True
    finally:
        if ok:                                             # on an error the peer may be gone: no rendezvous, just leave
            dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_nccl_sharding():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:                                        # never leave a rank (and its kernels) behind
        p.kill()
        p.join()
    assert not alive and all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for r in range(world):
        err_seq, err_heads, ok_oracle = ret[r]
        # the split result is the unsplit one up to the order of the partial sums
        assert err_seq < 2e-4, f"sequence split differs from the unsplit result by {err_seq}"
        assert ok_oracle, "sequence split outside the oracle tolerance"
        # heads packed alone quantise K over the same rows, so the result is the same up to
        # the fused kernel's own accumulation order
        assert err_heads < 2e-3, f"head sharding differs by {err_heads}"
