"""Torch-only restatement of the reference's TGN step, used by the end-to-end loss test (test infrastructure).

The dense math stays PyTorch in this project; this file only exists so that the data path (sampling, relabel,
gathers, state write-back) can be exercised under a real model.  Formulas follow the reference:
TimeEncoder (starrygl/nn/model/time_encoder.py:7-31), TransfomerAttentionLayer.forward
(starrygl/nn/gnn/graphattention.py:73-108, with ``edge_softmax`` / ``update_all`` written as index ops because DGL
is not available), GRU memory update from the mailbox (starrygl/nn/model/tgn.py:129-134, starrygl/nn/rnn/gru.py)
and EdgePredictor (starrygl/nn/model/EdgePredictor.py:2-25).
"""
import numpy as np
import torch
import torch.nn as nn


class TimeEncoder(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.w = nn.Linear(1, dim)
        self.w.weight = nn.Parameter(torch.from_numpy(1.0 / 10 ** np.linspace(0, 9, dim, dtype=np.float32)).reshape(dim, 1))
        self.w.bias = nn.Parameter(torch.zeros(dim))

    def forward(self, t):
        return torch.cos(self.w(t.float().reshape(-1, 1)))


class Attention(nn.Module):
    def __init__(self, dim_node, dim_edge, dim_time, heads, dim_out):
        super().__init__()
        self.h, self.dim_out = heads, dim_out
        self.time_enc = TimeEncoder(dim_time)
        self.w_q = nn.Linear(dim_node + dim_time, dim_out)
        self.w_k = nn.Linear(dim_node + dim_edge + dim_time, dim_out)
        self.w_v = nn.Linear(dim_node + dim_edge + dim_time, dim_out)
        self.w_out = nn.Linear(dim_node + dim_out, dim_out)
        self.norm = nn.LayerNorm(dim_out)
        self.act = nn.LeakyReLU(0.2)

    def forward(self, indptr, indices, x_src, x_dst, efeat, dt):
        """CSC block: dst row r owns edges indptr[r]:indptr[r+1]; ``indices`` point into x_src."""
        n_dst = indptr.numel() - 1
        dst_idx = torch.repeat_interleave(torch.arange(n_dst, device=indptr.device), indptr[1:] - indptr[:-1])
        inp = torch.cat((x_src[indices], efeat, self.time_enc(dt)), 1)
        query = torch.cat((x_dst, self.time_enc(torch.zeros(n_dst, device=indptr.device))), 1)
        Q = self.w_q(query).reshape(n_dst, self.h, -1)
        K = self.w_k(inp).reshape(inp.shape[0], self.h, -1)
        V = self.w_v(inp).reshape(inp.shape[0], self.h, -1)
        score = self.act((Q[dst_idx] * K).sum(2) / (self.dim_out // self.h) ** 0.5)
        # edge softmax over the in-edges of every destination
        mx = torch.full((n_dst, self.h), -1e30, device=score.device).scatter_reduce(0, dst_idx[:, None].expand_as(score), score,
                                                                                   "amax", include_self=True)
        ex = torch.exp(score - mx[dst_idx])
        den = torch.zeros(n_dst, self.h, device=score.device).index_add_(0, dst_idx, ex)
        att = ex / den[dst_idx]
        agg = torch.zeros(n_dst, self.dim_out, device=score.device).index_add_(0, dst_idx, (V * att[:, :, None]).reshape(V.shape[0], -1))
        return self.norm(torch.relu(self.w_out(torch.cat((agg, x_dst), 1))))


class TGN(nn.Module):
    def __init__(self, dim_mem, dim_edge, dim_time, heads=2):
        super().__init__()
        self.dim_mem = dim_mem
        self.mail_time = TimeEncoder(dim_time)
        self.gru = nn.GRUCell(2 * dim_mem + dim_edge + dim_time, dim_mem)
        self.att = Attention(dim_mem, dim_edge, dim_time, heads, dim_mem)
        self.src_fc, self.dst_fc, self.out_fc = nn.Linear(dim_mem, dim_mem), nn.Linear(dim_mem, dim_mem), nn.Linear(dim_mem, 1)

    def update_memory(self, mem, mem_ts, mail, mail_ts):
        return self.gru(torch.cat((mail, self.mail_time(mail_ts - mem_ts)), 1), mem)

    def forward(self, batch, n_events):
        """batch: dict of tensors produced by a data path (see test_gpu_tgn_e2e.py)."""
        x_dst = self.update_memory(batch["mem0"], batch["mem_ts0"], batch["mail0"], batch["mail_ts0"])
        x_src = self.update_memory(batch["mem1"], batch["mem_ts1"], batch["mail1"], batch["mail_ts1"])
        h = self.att(batch["indptr"], batch["indices"], x_src, x_dst, batch["efeat"], batch["edge_dt"])
        h = h[batch["inv_map"]]                       # one embedding per root, order cat(src, dst, neg)
        hs, hd, hn = h[:n_events], h[n_events:2 * n_events], h[2 * n_events:]
        pos = self.out_fc(torch.relu(self.src_fc(hs) + self.dst_fc(hd)))
        neg = self.out_fc(torch.relu(self.src_fc(hs) + self.dst_fc(hn)))
        loss = nn.functional.binary_cross_entropy_with_logits(pos, torch.ones_like(pos)) + \
            nn.functional.binary_cross_entropy_with_logits(neg, torch.zeros_like(neg))
        return loss, x_dst
