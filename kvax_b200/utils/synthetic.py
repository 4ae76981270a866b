"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations.  TEST / BENCH INFRASTRUCTURE (pure NumPy, no device code).

The reference measures on synthetic data only (kvax/utils/benchmarking.py:36-184:
N(0,1) bf16 tensors, piecewise-constant segment ids, PAD at the tail of each row), so
these generators are the workload rather than a stand-in for a dataset.  Differences
from the reference generator, on purpose: document lengths are log-uniform and
positions restart at 0 in every document, as the benchmark configurations ask.

Draw order per call is fixed: document lengths and pad counts row by row first, then
Q, K, V, dO.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

PADDING_SEGMENT_ID = -1


@dataclass(frozen=True)
class Config:
    name: str
    batch: int
    seq: int
    hq: int
    hkv: int
    head_dim: int
    tile: int
    doc_min: int
    doc_max: int
    pad_lo: float
    pad_hi: float
    dtype: str = "bf16"


CONFIGS = {
    # tiny case the CPU path can run in full
    "c1_tiny": Config("c1_tiny", 1, 512, 4, 2, 64, 64, 0, 0, 32 / 512, 32 / 512, "fp32"),
    # Llama-3-8B attention shape
    "c2_llama8b_8k": Config("c2_llama8b_8k", 1, 8192, 32, 8, 128, 128, 128, 4096, 0.0, 0.05),
    # dense causal limit: one document, no padding, MHA
    "c3_dense_causal_16k": Config("c3_dense_causal_16k", 4, 16384, 16, 16, 128, 128, 16384, 16384, 0.0, 0.0),
    # long-sequence document mask, the configuration the headline metric is quoted on
    "c4_docmask_32k": Config("c4_docmask_32k", 2, 32768, 32, 8, 128, 128, 256, 16384, 0.10, 0.10),
    # a dense causal case small enough for profiler captures (inputs still exceed no cache
    # budget that matters: K+V per head are streamed from L2/HBM)
    "profile_dense_8k": Config("profile_dense_8k", 2, 8192, 16, 16, 128, 128, 8192, 8192, 0.0, 0.0),
    "profile_dense_16k": Config("profile_dense_16k", 1, 16384, 16, 16, 128, 128, 16384, 16384, 0.0, 0.0),
    # context-parallel Llama-3-70B attention shape
    "c5_cp_128k": Config("c5_cp_128k", 1, 131072, 64, 8, 128, 128, 1024, 65536, 0.0, 0.0),
}


def document_layout(cfg: Config, rng: np.random.Generator, restart_positions: bool = True):
    """Returns int32 (positions, segment_ids), each (batch, seq)."""
    pos = np.zeros((cfg.batch, cfg.seq), np.int32)
    seg = np.full((cfg.batch, cfg.seq), PADDING_SEGMENT_ID, np.int32)
    for b in range(cfg.batch):
        frac = cfg.pad_lo if cfg.pad_hi == cfg.pad_lo else rng.uniform(cfg.pad_lo, cfg.pad_hi)
        n_pad = int(round(frac * cfg.seq))
        real = cfg.seq - n_pad
        if cfg.name == "c1_tiny":  # three documents from two distinct cut points
            cuts = np.sort(rng.choice(np.arange(1, real), size=2, replace=False))
            edges = [0, int(cuts[0]), int(cuts[1]), real]
        else:
            edges = [0]
            while edges[-1] < real:
                if cfg.doc_min >= cfg.doc_max:
                    n = cfg.doc_max
                else:
                    n = int(math.floor(math.exp(rng.uniform(math.log(cfg.doc_min), math.log(cfg.doc_max)))))
                edges.append(min(real, edges[-1] + max(n, 1)))
        for d, (s, e) in enumerate(zip(edges[:-1], edges[1:])):
            seg[b, s:e] = d
            pos[b, s:e] = np.arange(e - s) if restart_positions else np.arange(s, e)
        pos[b, real:] = np.arange(n_pad) if restart_positions else np.arange(real, cfg.seq)
    return pos, seg


def make_inputs(cfg: Config, seed: int = 0, restart_positions: bool = True, with_tensors: bool = True):
    """dict with positions, segment_ids, scale and (optionally) fp32 q, k, v, dout in the
    public (B, S, H, D) layout.  Callers cast to the compute dtype."""
    rng = np.random.default_rng(seed)
    pos, seg = document_layout(cfg, rng, restart_positions)
    out = dict(positions=pos, segment_ids=seg, scale=1.0 / math.sqrt(cfg.head_dim), cfg=cfg)
    if with_tensors:
        shp_q = (cfg.batch, cfg.seq, cfg.hq, cfg.head_dim)
        shp_kv = (cfg.batch, cfg.seq, cfg.hkv, cfg.head_dim)
        out["q"] = rng.standard_normal(shp_q, dtype=np.float32)
        out["k"] = rng.standard_normal(shp_kv, dtype=np.float32)
        out["v"] = rng.standard_normal(shp_kv, dtype=np.float32)
        out["dout"] = rng.standard_normal(shp_q, dtype=np.float32)
    return out


def small_config(name="small", batch=2, seq=1024, hq=4, hkv=2, head_dim=128, tile=128,
                 doc_min=64, doc_max=700, pad=0.07) -> Config:
    """A down-scaled case for parity tests the CPU oracle finishes in seconds."""
    return Config(name, batch, seq, hq, hkv, head_dim, tile, doc_min, doc_max, pad, pad)


def attention_flops(n_tiles: int, hq: int, d_qk: int, d_v: int, tile: int = 128):
    """Forward FLOPs for `n_tiles` visited tile pairs of one batch entry times `hq`
    heads, using the convention of kvax/utils/math.py:18-26 (2*(Dqk+Dv) per score
    element; backward = 2.5x, forward+backward = 3.5x)."""
    return 2.0 * (d_qk + d_v) * tile * tile * n_tiles * hq
