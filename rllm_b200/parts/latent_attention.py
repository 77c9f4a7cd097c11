"""Causal attention through low-rank latents (queries through one, keys and values through another),
with one rotated key part shared by all heads.

For input rows h [n, d] (H heads; per head dq plain and r rotated query/key entries, values of size
dv; latents of q_rank and kv_rank entries):

    cq = RMSNorm(h Wdq^T) (weight dq.norm);  q = cq Wuq^T, head by head [plain (dq) | rotated (r)]
    low = h Wdkv^T  [kv_rank + r];  c = RMSNorm(low[:kv_rank]) (weight dkv.norm);  kr = low[kv_rank:]
    the rotated parts (of every query head, and kr) get the rotary encoding over all r entries
    per head:  k_plain = Wuk_head c,  v = Wuv_head c
    s = (q_plain . k_plain + q_rot . kr) * scale;  p = softmax over the keys j <= i;  a = sum p_j v_j
    out = (a_1 | ... | a_H) Wo^T

Only [c | kr] is cached: one row of kv_rank + r entries per token and layer, whatever H is.  The
per-head keys and values are never formed: since q_plain . (Wuk c) = (Wuk^T q_plain) . c and
sum p_j (Wuv c_j) = Wuv (sum p_j c_j), the queries are taken into latent space (one small product
per head), attention runs with ONE key/value head whose keys are the cache rows and whose values
are the first kv_rank entries of the same rows, and Wuv is applied to the H results.

With `q_rank` 0 the queries have no latent: q = h Wq^T (tensor q in place of dq, dq.norm and uq).  With
`window` > 0 a token sees its last `window` keys only (itself included), and the cache gives back the pages
the window has passed.  The rotation's pair layout is the position part's.

Parameters: hidden_size, num_heads, head_dim, rot_dim, v_head_dim, kv_rank, q_rank, eps, scale,
softcap, window.  Tensors <prefix>dq, dq.norm, uq (or q), dkv, dkv.norm, uk, uv, o.  Load-time transforms: dq and
dkv are stacked into one product on h; uk is kept per head and transposed ([H, kv_rank, dq]).
Norms, angles, scores and softmax are float32 in every mode.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PagedKVNeed, PartError, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.H, self.dq, self.r = int(p["num_heads"]), int(p["head_dim"]), int(p["rot_dim"])
        self.dv, self.rank, self.q_rank = int(p["v_head_dim"]), int(p["kv_rank"]), int(p["q_rank"])
        self.eps = float(p.get("eps", 1e-6))
        self.scale = float(p["scale"])
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.window = int(p.get("window", 0) or 0)
        if self.r <= 0 or self.r % 2:
            raise PartError(f"latent_attention: rot_dim {self.r} must be positive and even")
        if self.rank > 512 or self.rank + self.r > 2048:
            raise PartError("latent_attention: kv_rank up to 512, kv_rank + rot_dim up to 2048")
        self.w_down = self.w_uq = self.w_qc = self.w_uv = self.w_o = self.q_norm_w = self.kv_norm_w = None

    def cache_need(self):
        return PagedKVNeed(1, self.rank + self.r, window=self.window, values_in_keys=self.rank)

    def expected_tensors(self):
        d, p, H = self.hidden_size, self.prefix, self.H
        q = ({p + "dq": ((self.q_rank, d), "matrix"), p + "dq.norm": ((self.q_rank,), "norm"),
              p + "uq": ((H * (self.dq + self.r), self.q_rank), "matrix")} if self.q_rank
             else {p + "q": ((H * (self.dq + self.r), d), "matrix")})
        return {**q, p + "dkv": ((self.rank + self.r, d), "matrix"), p + "dkv.norm": ((self.rank,), "norm"),
                p + "uk": ((H * self.dq, self.rank), "matrix"), p + "uv": ((H * self.dv, self.rank), "matrix"),
                p + "o": ((d, H * self.dv), "matrix")}

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        if self.q_rank:
            self.w_down = self._to_device(torch.cat([tensors[p + "dq"].to(dt), tensors[p + "dkv"].to(dt)], 0))
            self.q_norm_w = self._to_device(tensors[p + "dq.norm"], torch.float32)
            self.w_uq = self._to_device(tensors[p + "uq"])
        else:
            self.w_down = self._to_device(tensors[p + "dkv"])
            self.w_uq = self._to_device(tensors[p + "q"])
        self.kv_norm_w = self._to_device(tensors[p + "dkv.norm"], torch.float32)
        # [H, dq, rank] -> [H, rank, dq]: the product that takes a head's plain query into latent space
        self.w_qc = self._to_device(tensors[p + "uk"].to(dt).view(self.H, self.dq, self.rank).transpose(1, 2))
        self.w_uv = self._to_device(tensors[p + "uv"].to(dt).view(self.H, self.dv, self.rank))
        self.w_o = self._to_device(tensors[p + "o"])

    def forward(self, h, ctx, cache, position=None, residual=None):
        n, dt, dev = h.shape[0], self.runtime.dtype, h.device
        H, dq, r, rank = self.H, self.dq, self.r, self.rank
        if position is None or position.dims != r:
            raise PartError("latent_attention: needs a rotary position part over rot_dim entries")
        low = ops.linear(h, self.w_down, out_dtype=torch.float32)              # [query latent | c | kr]
        if self.q_rank:
            cq = torch.empty((n, self.q_rank), dtype=dt, device=dev)
            ops.norm_rows(low[:, :self.q_rank], self.q_norm_w, self.eps, low=cq)
            q = ops.linear(cq, self.w_uq, out_dtype=dt)                         # [n, H * (dq + r)]
        else:
            q = ops.linear(h, self.w_uq, out_dtype=dt)
        W = rank + r
        q_att = torch.empty((n, H * W), dtype=dt, device=dev)
        ops.head_linear(q.view(n, H, dq + r)[:, :, :dq], self.w_qc, q_att.view(n, H, W)[:, :, :rank])
        ops.latent_rope_store(q, low[:, self.q_rank:], self.kv_norm_w, position.angles(ctx), position.mult,
                              cache.slots, q_att, cache.k, H, dq, r, rank, cache.block_size, self.eps,
                              write_kv=cache.write, pairs=getattr(position, "layout", "half") == "pairs")
        mixed = torch.empty((n, H * rank), dtype=dt, device=dev)
        ops.shared_kv_attention(q_att, cache.k, mixed, ctx, cache.block_table, H, W, rank, cache.block_size,
                                self.scale, softcap=self.softcap, window=self.window)
        a = torch.empty((n, H * self.dv), dtype=dt, device=dev)
        ops.head_linear(mixed.view(n, H, rank), self.w_uv, a.view(n, H, self.dv))
        return ops.linear(a, self.w_o, out_dtype=torch.float32)
