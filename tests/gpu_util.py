import os

import numpy as np
import torch

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return np.load(os.path.join(G, name))


def cu(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def npy(t):
    return t.detach().cpu().numpy()


def build_graph(z, keyed_by="dst"):
    """T-CSR on the GPU with the oracle's roles (rows keyed by dst, neighbour = src) unless asked otherwise."""
    from starrygl import ops
    key, nbr = (z["dst"], z["src"]) if keyed_by == "dst" else (z["src"], z["dst"])
    return ops.tcsr_build(cu(key), cu(nbr), cu(z["ts"]), cu(z["eid"]), int(z["n"]), want_perm=True)
