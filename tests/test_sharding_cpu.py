"""Host-side sharding logic on 2 gloo ranks (CPU): head slices, token slices, the
all-gather + log-sum-exp combine of sequence-split records (oracle as the compute),
and the group consistency check."""
import datetime
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
    # row windows: disjoint, in order, covering [0, rows), starting on multiples of 64
    for rows, parts in ((2048, 2), (1000, 3), (77, 1), (60, 4), (8192, 8)):
        w = [sharding.row_window(p, parts, rows) for p in range(parts)]
        assert w[0][0] == 0 and w[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(w, w[1:])) and all(lo % 64 == 0 or lo == rows for lo, _ in w)
    with pytest.raises(ValueError):
        sharding.row_window(2, 2, 100)
    # parts of a head: every phase shared out, cut points on multiples of 32 rows, nothing lost
    for counts in ((512, 768, 512, 256), (100, 0, 37, 5), (31, 33, 64, 1)):
        for parts in (1, 2, 3):
            got = [sharding.part_rows(counts, p, parts) for p in range(parts)]
            base = 0
            for ph, n in enumerate(counts):
                spans = [got[p][ph] for p in range(parts)]
                assert spans[0][0] == base and spans[-1][1] == base + n
                assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
                assert all((lo - base) % 32 == 0 for lo, _ in spans)
                base += n


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, mode, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
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
            # ONE packed layer (the reference's); every rank attends over its window of each head's
            # live rows (ragged heads: the windows cut them at different places), then the records are merged
            vb = synth.make_v_bits(H_kv, T, N, seed=seed, per_head_N=[96, 40, 77, 64])
            layer, nv = RP.pack_kv(K.numpy(), V.numpy(), vb.numpy(), kb.numpy(), g)
            o, m, l = RA.decode_attention(q, layer, nv, seq_part=(rank, world))
            rec = np.zeros((H_kv * g, 132), np.float32)
            rec[:, 0], rec[:, 1], rec[:, 4:] = m, l, o * l[:, None]

            def combine(records):
                r = records.numpy()
                out, _, _ = RA.lse_combine(r[:, :, 0].T, r[:, :, 1].T, r[:, :, 4:].transpose(1, 0, 2))
                return torch.from_numpy(out)

            sharding.check_group_consistency(rec.shape[0])
            got = sharding.combine_across_ranks(torch.from_numpy(rec), combine=combine).numpy()
            want = RA.decode_attention(q, layer, nv)[0]      # the unsplit result
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
        p.daemon = True
        p.start()
    for p in procs:
        p.join(120)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:                                        # never leave a rank behind
        p.kill()
        p.join()
    assert not alive and all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    if mode == "mismatch":
        assert all(ret[r] == "ValueError" for r in range(world))
    else:
        assert all(ret[r] < 1e-5 for r in range(world)), dict(ret)
