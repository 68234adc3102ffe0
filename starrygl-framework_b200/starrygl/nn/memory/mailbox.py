"""Mailbox of the memory module: per node ``mailbox_size`` slots of ``[own state | other end's state | edge feature]``
rows with their timestamps (reference: starrygl/nn/memory/mailbox.py:5-107).

Same class name, constructor and method names as the reference.  The work is done by two library kernels chains:
``ops.mail_reduce`` (latest message per node + row assembly, replaces cat / unique / scatter_max / index of
``get_update_mail``) and ``ops.mailbox_write`` (the indexed writes and ring-position update of
``set_mailbox_local``).  There is no CPU path: the mailbox lives on the GPU from construction.

Differences from the reference, all on paths it cannot run as committed: ``set_mailbox_local`` there reads
``self.num_parts``, ``self.memory_param`` and ``.accessor`` attributes that the class never sets; here the reduce
is applied when ``Reduce_Op == 'max'`` (any world size) and the slot count is ``self.mailbox_size``.  Ties between
equal timestamps of one node resolve to the FIRST entry (the order of the strict ``>`` update of a sequential
scatter-max); the reference's GPU scatter is unordered there.
"""
from typing import Optional

import torch

from ... import _C, ops
from ...utils.context import DistributedContext


class mailbox:
    def __init__(self, num_nodes, mailbox_size, dim_out, dim_edge_feat, _next_mail_pos=None, _update_mail_pos=False,
                 device=None):
        if device is None:
            device = DistributedContext.get_default_context().device
        device = torch.device(device)
        if device.type != "cuda":
            raise _C.SglError("mailbox: the data path has no CPU implementation, pass a CUDA device")
        self.num_nodes, self.mailbox_size = int(num_nodes), int(mailbox_size)
        self.dim_out, self.dim_edge_feat = int(dim_out), int(dim_edge_feat)
        self.device = device
        self.mailbox = torch.zeros(self.num_nodes, self.mailbox_size, 2 * self.dim_out + self.dim_edge_feat,
                                   device=device, dtype=torch.float32)
        self.mailbox_ts = torch.zeros((self.num_nodes, self.mailbox_size), dtype=torch.float32, device=device)
        self.next_mail_pos = (torch.zeros(self.num_nodes, dtype=torch.long, device=device) if _next_mail_pos is None
                              else _next_mail_pos.to(device))
        self.update_mail_pos = _update_mail_pos
        self._status = ops.StatusWord(device)

    @property
    def shape(self):
        return (self.num_nodes, self.mailbox_size, 2 * self.dim_out + self.dim_edge_feat)

    @property
    def status(self):
        return self._status

    def reset(self):
        self.mailbox.fill_(0)
        self.mailbox_ts.fill_(0)
        self.next_mail_pos.fill_(0)

    def move_to_gpu(self):
        """Kept for call compatibility: the mailbox is created on the GPU."""
        return self

    # ---- latest message per node -------------------------------------------------------------------------------
    def get_update_mail_async(self, src, dst, ts, edge_feats, mem_src, mem_dst, embedding=None, use_src_emb=False,
                              use_dst_emb=False):
        """``get_update_mail`` without the host synchronisation: returns ``(index, mail, mail_ts, d_n)`` where the
        tensors have capacity ``2 * len(src)`` and the device scalar ``d_n`` holds the number of distinct nodes."""
        src, dst = src.to(self.device), dst.to(self.device)
        n = src.numel()
        emb_src = emb_dst = None
        if embedding is not None:
            emb_src, emb_dst = embedding[:n], embedding[n:]
        f = lambda t: t.to(self.device, torch.float32).contiguous()
        a1, a2 = f(emb_src if use_src_emb else mem_src), f(emb_dst if use_dst_emb else mem_dst)
        b1, b2 = f(emb_dst if use_src_emb else mem_dst), f(emb_src if use_dst_emb else mem_src)
        segs = [(a1, b1), (a2, b2)]
        if edge_feats is not None:
            ef = f(edge_feats)
            segs.append((ef, ef))
        ts = ts.to(self.device)
        if ts.dtype not in (torch.int64, torch.float32):
            ts = ts.to(torch.float32)
        index, mail, mail_ts, _, d_n = ops.mail_reduce(src.reshape(-1), dst.reshape(-1), ts.reshape(-1), self.num_nodes, segs,
                                                       status=self._status)
        return index, mail, mail_ts, d_n

    def get_update_mail(self, src, dst, ts, edge_feats, mem_src, mem_dst, embedding=None, use_src_emb=False,
                        use_dst_emb=False, block=None, Reduce_score=None):
        """(index, mail, mail_ts) of the batch: distinct nodes in ascending order, each with the row and timestamp of
        its latest entry (reference: mailbox.py:56-84).  One host synchronisation, to size the results exactly."""
        index, mail, mail_ts, d_n = self.get_update_mail_async(src, dst, ts, edge_feats, mem_src, mem_dst, embedding,
                                                               use_src_emb, use_dst_emb)
        u = int(d_n.item())
        return index[:u], mail[:u], mail_ts[:u]

    # ---- writes ------------------------------------------------------------------------------------------------
    def set_mailbox_local(self, index, source, source_ts, Reduce_Op=None, d_n=None):
        """``mailbox[index, next_mail_pos[index]] = source`` (+ timestamps), then the ring position of those nodes
        advances (reference: mailbox.py:41-54).  ``Reduce_Op == 'max'`` first keeps the latest row per distinct node.
        Without the reduce ``index`` must hold distinct nodes."""
        index = index.to(self.device)
        source = source.to(self.device, torch.float32).contiguous()
        source_ts = source_ts.to(self.device)
        if Reduce_Op == 'max':
            if d_n is not None:
                raise _C.SglError("set_mailbox_local: a device-side count cannot be combined with Reduce_Op")
            ts = source_ts if source_ts.dtype in (torch.int64, torch.float32) else source_ts.to(torch.float32)
            index, source, source_ts, _, d_n = ops.mail_reduce(index.reshape(-1), None, ts.reshape(-1), self.num_nodes,
                                                               [(source, None)], status=self._status)
        else:
            source_ts = source_ts.to(torch.float32)
        ops.mailbox_write(index, source, source_ts.contiguous(), self.mailbox, self.mailbox_ts, self.next_mail_pos, d_n=d_n,
                          advance=self.mailbox_size > 1, status=self._status)

    def update_mailbox(self, index, mail, mail_ts, d_n=None):
        """Name the reference's training loop calls (test/test.py:328); same as ``set_mailbox_local``."""
        self.set_mailbox_local(index, mail, mail_ts, d_n=d_n)

    def update_next_mail_pos(self):
        if self.update_mail_pos is not None and torch.is_tensor(self.update_mail_pos):
            nid = torch.where(self.update_mail_pos == 1)[0]
            self.next_mail_pos[nid] = torch.remainder(self.next_mail_pos[nid] + 1, self.mailbox_size)
            self.update_mail_pos.fill_(0)

    # ---- reads -------------------------------------------------------------------------------------------------
    def get_message(self, idx):
        """(mailbox[idx], mailbox_ts[idx]) through the row-gather kernel."""
        idx = idx.to(self.device)
        n, s, w = self.shape
        rows = ops.gather_rows(self.mailbox.view(n, s * w), idx, status=self._status).view(-1, s, w)
        ts = ops.gather_rows(self.mailbox_ts, idx, status=self._status)
        return rows, ts
