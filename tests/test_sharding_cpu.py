"""Host-side sharding logic on 2 gloo ranks (CPU): head slices, token slices, the
all-gather + log-sum-exp combine of sequence-split records (oracle as the compute),
and the group consistency check."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rdkv_b200 import sharding, synth


def test_head_shard_and_grid():
    assert [sharding.head_shard(r, 4, 8) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert sharding.head_shard(0, 1, 8) == (0, 8)
    with pytest.raises(ValueError):
        sharding.head_shard(0, 3, 8)
    with pytest.raises(ValueError):
        sharding.head_shard(4, 4, 8)
    assert sharding.grid(5, 8, 2) == (2, 4, 1)
    with pytest.raises(ValueError):
        sharding.grid(0, 6, 4)
    vb = synth.make_v_bits(2, 64, 32, seed=3)
    parts = [sharding.split_tokens(vb, p, 2) for p in range(2)]
    assert torch.equal(parts[0] + parts[1], vb) and int((parts[0][:, 32:] != 0).sum()) == 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, mode, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import ref_attention as RA
        from oracle import ref_packing as RP
        H_kv, g, T, N = 4, 2, 256, 96
        seed = synth.unit_seed(4, 1, 0)
        K, V = synth.make_kv(H_kv, T, seed=seed)
        vb = synth.make_v_bits(H_kv, T, N, seed=seed)
        kb = synth.make_k_bits(H_kv, seed=seed)
        q = synth.make_q(H_kv * g, seed=seed + 1).numpy()
        if mode == "sequence":
            # every rank packs its token slice of all heads, then the records are merged
            mine = sharding.split_tokens(vb, rank, world)
            layer, nv = RP.pack_kv(K.numpy(), V.numpy(), mine.numpy(), kb.numpy(), g)
            o, m, l = RA.decode_attention(q, layer, nv)
            rec = np.zeros((H_kv * g, 132), np.float32)
            rec[:, 0], rec[:, 1], rec[:, 4:] = m, l, o * l[:, None]

            def combine(records):
                r = records.numpy()
                out, _, _ = RA.lse_combine(r[:, :, 0].T, r[:, :, 1].T, r[:, :, 4:].transpose(1, 0, 2))
                return torch.from_numpy(out)

            sharding.check_group_consistency(rec.shape[0])
            got = sharding.combine_across_ranks(torch.from_numpy(rec), combine=combine).numpy()
            # expected: attention over the union of both slices' dequantised rows
            halves = []
            for p in range(world):
                lp, nvp = RP.pack_kv(K.numpy(), V.numpy(), sharding.split_tokens(vb, p, world).numpy(), kb.numpy(), g)
                halves.append(RA.decode_attention(q, lp, nvp))
            want, _, _ = RA.lse_combine(np.stack([h[1] for h in halves]), np.stack([h[2] for h in halves]),
                                        np.stack([h[0] * h[2][:, None] for h in halves]))
            ret[rank] = float(np.abs(got - want).max())
        elif mode == "heads":
            Ks, Vs, vbs, kbs = sharding.shard_heads(K, V, vb, kb, rank, world)
            layer, nv = RP.pack_kv(Ks.numpy(), Vs.numpy(), vbs.numpy(), kbs.numpy(), g)
            h0, h1 = sharding.head_shard(rank, world, H_kv)
            o, _, _ = RA.decode_attention(q[h0 * g:h1 * g], layer, nv)
            full_layer, full_nv = RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g)
            # a head packed alone sees the same stripe only if extents agree; compare through gather
            outs = [torch.zeros(o.shape) for _ in range(world)]
            dist.all_gather(outs, torch.from_numpy(o))
            got = torch.cat(outs).numpy()
            want = np.concatenate([RA.decode_attention(
                q[r * (H_kv // world) * g:(r + 1) * (H_kv // world) * g],
                *RP.pack_kv(*[t.numpy() for t in sharding.shard_heads(K, V, vb, kb, r, world)], g))[0]
                for r in range(world)])
            ret[rank] = float(np.abs(got - want).max())
        elif mode == "mismatch":
            try:
                sharding.check_group_consistency(8 + rank)
                ret[rank] = "no error"
            except ValueError as e:
                ret[rank] = "ValueError"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["sequence", "heads", "mismatch"])
def test_two_rank_gloo(mode):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    if mode == "mismatch":
        assert all(ret[r] == "ValueError" for r in range(world))
    else:
        assert all(ret[r] < 1e-5 for r in range(world)), dict(ret)
