"""Slot files written by the GPU builder (``starrygl.graph.materialize``) against the files the reference's
``build_aligned_batch`` wrote for the same partitions and tasks (golden ``slots.npz``): same keys, same tensors, same
per-layer route plans (inside a destination-rank segment the reference's order comes from an unstable argsort, so
segments are compared as multisets)."""
import os

import numpy as np
import pytest
import torch

from gpu_util import load
from test_oracle_golden import LAYER_KEYS, same_plan_up_to_segment_order, slot_cases

pytestmark = pytest.mark.gpu


def test_slot_files_match_the_reference(tmp_path):
    from starrygl.cache.replica_table import CSRReplicaTable
    from starrygl.graph.materialize import MaterializedMultiLayerBuilder
    builders = {}
    for z, c, pid, roots, rts in slot_cases():
        if pid not in builders:
            rt = CSRReplicaTable(torch.from_numpy(z["rt_indptr"]), torch.from_numpy(z["rt_ranks"]), torch.from_numpy(z["rt_locs"]))
            builders[pid] = MaterializedMultiLayerBuilder({k: z[k] for k in ("src", "dst", "ts", "eid")}, int(z["N"]),
                                                          torch.from_numpy(z["node_parts"]), rt, pid, int(z["P"]))
        pick = z[f"c{c}_pick"]
        kind = str(z[f"c{c}_kind"])
        if kind == "link":
            task = ('link', (z["src"][pick], z["dst"][pick], z["ts"][pick], np.ones(len(pick), np.int64), z["eid"][pick]))
        else:
            task = ('node', (z["dst"][pick], z["ts"][pick], np.zeros(len(pick), np.int64)))
        cfg = {'meta': {'start_offset': -1, 'end_offset': int(z[f"c{c}_end_offset"]), 'graph_type': 'c'},
               'layer': [{'type': 'recent', 'fanout': int(f)} for f in z[f"c{c}_fanouts"]]}
        path = os.path.join(tmp_path, f"slot_{c:04d}_sub_{pid:04d}.pt")
        builders[pid].build_aligned_batch(task, path, cfg, 1, None, None)
        data = torch.load(path, weights_only=False)          # what a loader of the reference would read
        tag = f"c{c}_p{pid}"
        assert len(data) == int(z[f"{tag}_num_layers"])
        ref_keys = {f[len(tag) + 4:] for f in z.files if f.startswith(f"{tag}_L0_")}
        assert ref_keys <= set(data[0].keys()) and "comm_plan" in data[0], (tag, ref_keys - set(data[0].keys()))
        for k in ref_keys:
            v = data[0][k]
            assert not (torch.is_tensor(v) and v.is_cuda)
            assert np.array_equal(np.asarray(v), z[f"{tag}_L0_{k}"]), (tag, k)
        for i in range(1, len(data)):
            assert set(data[i].keys()) == set(LAYER_KEYS)
            for k in LAYER_KEYS:
                a, r = data[i][k].numpy(), z[f"{tag}_L{i}_{k}"]
                assert a.dtype == r.dtype and np.array_equal(a, r), (tag, i, k)
        plans = data[0]["comm_plan"]
        assert len(plans) == int(z[f"{tag}_num_plans"])
        for i, pl in enumerate(plans):
            got = None if pl is None else (pl.send_ranks.numpy(), pl.send_sizes.numpy(), pl.send_indices.numpy(),
                                           pl.send_remote_indices.numpy())
            assert same_plan_up_to_segment_order(got, z, f"{tag}_plan{i}"), (tag, i)


def test_unsupported_policies_raise():
    from starrygl.graph.materialize import MaterializedMultiLayerBuilder
    e = np.arange(4, dtype=np.int64)
    b = MaterializedMultiLayerBuilder({'src': e, 'dst': e[::-1].copy(), 'ts': e}, 4, None, None, 0, 1)
    task = ('node', (e, e + 10, e))
    for cfg in ({'meta': {'graph_type': 'd'}, 'layer': [{'type': 'recent', 'fanout': 2}]},
                {'meta': {}, 'layer': [{'type': 'cluster', 'fanout': 2}]},
                {'meta': {'end_offset': 5}, 'layer': [{'type': 'recent', 'fanout': 2}]}):
        with pytest.raises(NotImplementedError):
            b.build_aligned_batch(task, None, cfg)
    out = b.build_aligned_batch(task, None, {'meta': {}, 'layer': [{'type': 'uniform', 'fanout': 2}]}, seed=3)
    assert out[0]["comm_plan"] == [None, None] and out[1]["indptr"].numel() == out[0]["gids"].numel() + 1
