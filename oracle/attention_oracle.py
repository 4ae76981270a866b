"""CPU oracle for document-masked causal GQA attention.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline / reference arm of the benchmark
may import this module; the product path never does.

Restates the dense masked attention the reference's tests compare their kernels with:
  tests/test_attention.py:33-49            dense mask = (q_seg == kv_seg) & (q_pos >= kv_pos)
  kvax/ops/flash_attention_cudnn.py:14-24  segment mask
  kvax/ops/flash_attention_cudnn.py:91-113 softmax(scale * Q K^T + mask) V with KV heads
                                           shared by Hq/Hkv query heads
The dense op itself is jax.nn.dot_product_attention (third-party, jax>=0.4.34 per the
reference's pyproject.toml, not vendored and not installed here) so its published
definition is restated.

Parity is pinned: tests/golden/attn_*.npz hold the outputs of the reference's own
`flash_attention_triton_forward` and `flash_attention_backward` (host code and Triton
kernels, run by Triton's CPU interpreter through tests/golden/make_attention_golden.py) on
eight small seeded cases (GQA and MHA, head_dim 64 / 128, restarting and global positions,
`assume_sequential_positions`, mixed block sizes, ragged lengths, decode, the two ranks of a
context-parallel run);
tests/test_oracle_attention.py checks this restatement against them to 2e-5 for O, LSE2,
dQ, dK and dV on every row the reference specifies.

Layouts follow the public API: q (B, Sq, Hq, D), k/v (B, Skv, Hkv, D).
"""
from __future__ import annotations

import numpy as np

PADDING_SEGMENT_ID = -1


def _mask(q_pos, q_seg, kv_pos, kv_seg):
    return (q_seg[:, :, None] == kv_seg[:, None, :]) & (q_pos[:, :, None] >= kv_pos[:, None, :])


def attention_forward(q, k, v, q_pos, q_seg, kv_pos, kv_seg, scale, dtype=np.float64):
    """Returns (out (B,Sq,Hq,Dv), lse2 (B,Hq,Sq)) — lse2 is the base-2 log-sum-exp of
    the scaled scores, the quantity the reference's forward kernel stores
    (flash_attention_triton.py:366-369).  Rows with no unmasked key give out=0."""
    q = np.asarray(q, dtype); k = np.asarray(k, dtype); v = np.asarray(v, dtype)
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    mask = _mask(np.asarray(q_pos), np.asarray(q_seg), np.asarray(kv_pos), np.asarray(kv_seg))
    out = np.zeros((B, Sq, Hq, v.shape[3]), dtype)
    lse2 = np.zeros((B, Hq, Sq), dtype)
    for b in range(B):
        for h in range(Hq):
            s = (q[b, :, h] @ k[b, :, h // G].T) * scale
            s = np.where(mask[b], s, -np.inf)
            m = s.max(-1, keepdims=True)
            m = np.where(np.isfinite(m), m, 0.0)
            p = np.exp(s - m)
            l = p.sum(-1, keepdims=True)
            safe = np.where(l > 0, l, 1.0)
            out[b, :, h] = (p / safe) @ v[b, :, h // G]
            with np.errstate(divide="ignore"):
                lse2[b, h] = ((m + np.log(safe)) / np.log(2.0))[:, 0]
            lse2[b, h] = np.where(l[:, 0] > 0, lse2[b, h], np.inf)
    return out, lse2


def attention_backward(q, k, v, q_pos, q_seg, kv_pos, kv_seg, scale, dout, dtype=np.float64):
    """Analytic gradients of sum(out * dout) w.r.t. q, k, v (GQA: dk/dv summed over the
    query heads of a group, as flash_attention_triton.py:1855-1868 does)."""
    q = np.asarray(q, dtype); k = np.asarray(k, dtype); v = np.asarray(v, dtype)
    dout = np.asarray(dout, dtype)
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    mask = _mask(np.asarray(q_pos), np.asarray(q_seg), np.asarray(kv_pos), np.asarray(kv_seg))
    dq = np.zeros_like(q); dk = np.zeros_like(k); dv = np.zeros_like(v)
    for b in range(B):
        for h in range(Hq):
            g = h // G
            s = (q[b, :, h] @ k[b, :, g].T) * scale
            s = np.where(mask[b], s, -np.inf)
            m = s.max(-1, keepdims=True)
            m = np.where(np.isfinite(m), m, 0.0)
            p = np.exp(s - m)
            l = p.sum(-1, keepdims=True)
            p = p / np.where(l > 0, l, 1.0)
            do = dout[b, :, h]
            dv[b, :, g] += p.T @ do
            dp = do @ v[b, :, g].T
            delta = (p * dp).sum(-1, keepdims=True)
            ds = p * (dp - delta) * scale
            dq[b, :, h] = ds @ k[b, :, g]
            dk[b, :, g] += ds.T @ q[b, :, h]
    return dq, dk, dv


def attention_fwd_bwd_torch(q, k, v, q_pos, q_seg, kv_pos, kv_seg, scale, dout, heads_chunk=None):
    """Same computation with torch CPU ops (multi-threaded fp32) — the timed CPU baseline.
    Returns (out, dq, dk, dv) as torch tensors."""
    import torch

    q = torch.as_tensor(q, dtype=torch.float32).requires_grad_(True)
    k = torch.as_tensor(k, dtype=torch.float32).requires_grad_(True)
    v = torch.as_tensor(v, dtype=torch.float32).requires_grad_(True)
    dout = torch.as_tensor(dout, dtype=torch.float32)
    B, Sq, Hq, D = q.shape
    G = Hq // k.shape[2]
    q_pos = torch.as_tensor(q_pos); kv_pos = torch.as_tensor(kv_pos)
    q_seg = torch.as_tensor(q_seg); kv_seg = torch.as_tensor(kv_seg)
    mask = (q_seg[:, :, None] == kv_seg[:, None, :]) & (q_pos[:, :, None] >= kv_pos[:, None, :])
    kk = k.repeat_interleave(G, dim=2)
    vv = v.repeat_interleave(G, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
    s = s.masked_fill(~mask[:, None], float("-inf"))
    rowmax = s.amax(-1, keepdim=True)
    rowmax = torch.where(torch.isfinite(rowmax), rowmax, torch.zeros_like(rowmax))
    p = torch.exp(s - rowmax)
    l = p.sum(-1, keepdim=True)
    p = p / torch.where(l > 0, l, torch.ones_like(l))
    out = torch.einsum("bhqk,bkhd->bqhd", p, vv)
    (out * dout).sum().backward()
    return out.detach(), q.grad, k.grad, v.grad


def attention_dense_torch(q, k, v, q_pos, q_seg, kv_pos, kv_seg, scale, dout=None, kv_heads=None, batch_rows=None,
                          q_chunk=4096):
    """The same dense masked attention and its analytic gradients with torch fp32 ops, on whatever
    device the inputs live on, evaluated in blocks of `q_chunk` query rows against the key range
    their segment ids can match, so that sequences of 10^4 - 10^5 tokens fit in memory.  It is the
    fp32 reference of the parity tests at the benchmark sizes, where the NumPy loops above would
    take hours; tests/test_oracle_attention.py checks it against those loops on small cases.

    q (B, Sq, Hq, D), k / v (B, Skv, Hkv, D) tensors of any float dtype (computed in fp32; fp32
    matmuls must not be allowed to use tf32).  `kv_heads` / `batch_rows`: subsets to evaluate
    (default all); a kv head is always evaluated with all query heads of its group, because
    dk / dv sum over the group.  Returns a dict: out (B, Sq, Hq, Dv), lse2 (B, Hq, Sq) and, with
    `dout`, dq, dk, dv -- zeros outside the evaluated subsets -- plus the lists of evaluated
    batch rows, kv heads and query heads.  Key ranges are found from segment ids, which must be
    piecewise constant along the sequence (documents are contiguous), as everywhere in this repo.
    """
    import math

    import torch

    assert not torch.backends.cuda.matmul.allow_tf32
    dev = q.device
    B, Sq, Hq, D = q.shape
    Skv, Hkv, Dv = k.shape[1], k.shape[2], v.shape[3]
    G = Hq // Hkv
    kv_heads = list(range(Hkv)) if kv_heads is None else list(kv_heads)
    batch_rows = list(range(B)) if batch_rows is None else list(batch_rows)
    q_pos, q_seg, kv_pos, kv_seg = (torch.as_tensor(t).to(dev) for t in (q_pos, q_seg, kv_pos, kv_seg))
    out = torch.zeros((B, Sq, Hq, Dv), dtype=torch.float32, device=dev)
    lse2 = torch.zeros((B, Hq, Sq), dtype=torch.float32, device=dev)
    grads = dout is not None
    if grads:
        dq = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=dev)
        dk = torch.zeros((B, Skv, Hkv, D), dtype=torch.float32, device=dev)
        dv = torch.zeros((B, Skv, Hkv, Dv), dtype=torch.float32, device=dev)
    for b in batch_rows:
        for s in range(0, Sq, q_chunk):
            e = min(Sq, s + q_chunk)
            qs_, qp_ = q_seg[b, s:e], q_pos[b, s:e]
            # keys whose segment id occurs among this block's queries form one index range
            lo_id, hi_id = int(qs_.min()), int(qs_.max())
            cand = torch.nonzero((kv_seg[b] >= lo_id) & (kv_seg[b] <= hi_id))
            if cand.numel() == 0:
                continue
            k0, k1 = int(cand.min()), int(cand.max()) + 1
            mask = (qs_[:, None] == kv_seg[b, k0:k1][None, :]) & (qp_[:, None] >= kv_pos[b, k0:k1][None, :])
            for g in kv_heads:
                hs = slice(g * G, (g + 1) * G)
                qg = q[b, s:e, hs].float().permute(1, 0, 2)                     # (G, qc, D)
                kg, vg = k[b, k0:k1, g].float(), v[b, k0:k1, g].float()         # (kc, D)
                sc = torch.matmul(qg, kg.t()) * scale                           # (G, qc, kc)
                sc = sc.masked_fill(~mask[None], float("-inf"))
                m = sc.amax(-1, keepdim=True)
                m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
                p = torch.exp(sc - m)
                del sc
                l = p.sum(-1, keepdim=True)
                p = p / torch.where(l > 0, l, torch.ones_like(l))
                out[b, s:e, hs] = torch.matmul(p, vg).permute(1, 0, 2)
                l2 = (m + torch.log(torch.where(l > 0, l, torch.ones_like(l)))) / math.log(2.0)
                lse2[b, hs, s:e] = torch.where(l > 0, l2, torch.full_like(l2, float("inf")))[:, :, 0]
                if grads:
                    dog = dout[b, s:e, hs].float().permute(1, 0, 2)             # (G, qc, Dv)
                    dv[b, k0:k1, g] += torch.matmul(p.transpose(1, 2), dog).sum(0)
                    dp = torch.matmul(dog, vg.t())
                    delta = (p * dp).sum(-1, keepdim=True)
                    ds = p * (dp - delta) * scale
                    del dp
                    dq[b, s:e, hs] = torch.matmul(ds, kg).permute(1, 0, 2)
                    dk[b, k0:k1, g] += torch.matmul(ds.transpose(1, 2), qg).sum(0)
                    del ds
                del p
    res = dict(out=out, lse2=lse2, batch_rows=batch_rows, kv_heads=kv_heads,
               q_heads=[h for g in kv_heads for h in range(g * G, (g + 1) * G)])
    if grads:
        res.update(dq=dq, dk=dk, dv=dv)
    return res
