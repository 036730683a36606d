"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations: a plumbing case, a mixed-adapter decode batch over one transformer block, prefill
segments, heterogeneous ranks over one wide layer, and a tensor-parallel 27B-shaped layer.

Everything is numpy on the host; callers move it to the device. Adapter index i (0-based) lives in GPU
slot i + 1; slot 0 is "no adapter".
"""
import numpy as np

from .sites import Factors, Site, bf16_bits


def block_sites(hidden, inter, kv, layer=0):
    """The four adapter sites of one decoder layer in engine order (src/model.rs:684-786): fused q/k/v,
    attention out, fused gate/up, down."""
    return [
        Site.fused(layer, hidden, [("self_attn.q_proj", hidden), ("self_attn.k_proj", kv), ("self_attn.v_proj", kv)]),
        Site.fused(layer, hidden, [("self_attn.o_proj", hidden)]),
        Site.fused(layer, hidden, [("mlp.gate_proj", inter), ("mlp.up_proj", inter)]),
        Site.fused(layer, inter, [("mlp.down_proj", hidden)]),
    ]


class Workload:
    def __init__(self, name, sites, ranks, scale, row_n, row_slot, seed, max_rank=None, std=0.02):
        self.name = name
        self.sites = sites
        self.ranks = list(ranks)            # rank of adapter i
        self.scale = scale
        self.row_n = np.asarray(row_n, np.int32)      # tokens of each sequence, step order
        self.row_slot = np.asarray(row_slot, np.int32)  # GPU slot of each sequence (0 = base only)
        self.seed = seed
        self.std = std
        self.max_rank = max_rank or max(self.ranks)
        self.n_adapters = len(self.ranks)
        self.tokens = int(self.row_n.sum())
        self.n_seqs = len(self.row_n)

    def token_slot(self):
        return np.repeat(self.row_slot, self.row_n).astype(np.int32)

    def cu(self):
        return np.concatenate([[0], np.cumsum(self.row_n)]).astype(np.int32)

    def factors(self, i):
        """Adapter i's modules: A [r, cols] and scale * B [rows, r], drawn N(0, std^2) in f32."""
        r = self.ranks[i]
        out = []
        for si, site in enumerate(self.sites):
            for pi, part in enumerate(site.parts):
                rng = np.random.default_rng([self.seed, 1000 + i, si, pi])
                a = rng.standard_normal((r, site.cols), dtype=np.float32) * np.float32(self.std)
                b = rng.standard_normal((part.rows, r), dtype=np.float32) * np.float32(self.std)
                out.append(Factors.scaled(site.layer, part.module, a, b, self.scale))
        return out

    def x_bits(self, si):
        """The layer input of site si: [tokens, cols] ~ N(0, 1) as bf16 bit patterns."""
        rng = np.random.default_rng([self.seed, 1, si])
        return bf16_bits(rng.standard_normal((self.tokens, self.sites[si].cols), dtype=np.float32))

    def y_base(self, si):
        """Stand-in for the layer's own x W^T (an input of this path): [tokens, width] ~ N(0, 1), f32."""
        rng = np.random.default_rng([self.seed, 2, si])
        return rng.standard_normal((self.tokens, self.sites[si].width()), dtype=np.float32)

    # ---- algorithmic work of one pass over all sites, true ranks (bytes, flops) ----
    def work(self, f32_out=False):
        tslot = self.token_slot()
        present = np.unique(tslot[tslot > 0])
        t_by_slot = {int(s): int((tslot == s).sum()) for s in present}
        t_l = int((tslot > 0).sum())
        tiles = int(sum((n + 15) // 16 for n, s in zip(self.row_n, self.row_slot) if s != 0))
        ye = 8 if f32_out else 4
        by, fl = 0, 0
        parts = {"slabs": 0, "x": 0, "s": 0, "y": 0, "meta": 0}
        for site in self.sites:
            n_tot = sum(p.rows for p in site.parts)
            np_ = len(site.parts)
            for s, ta in t_by_slot.items():
                r = self.ranks[s - 1]
                parts["slabs"] += 2 * (np_ * r * site.cols + n_tot * r)
                parts["s"] += ta * np_ * r * 4 * 2
                parts["y"] += ta * n_tot * ye
                fl += ta * 2 * (np_ * r * site.cols + r * n_tot)
            parts["x"] += 2 * t_l * site.cols
            parts["meta"] += 4 + 12 * tiles + 112 * len(present)
        by = sum(parts.values())
        return {"bytes": by, "flops": fl, "parts": parts, "tokens": self.tokens, "lora_tokens": t_l,
                "slots_present": len(present), "tiles": tiles}


def config1(seed=0):
    """Plumbing: one bf16 layer 1024 -> 1024, 16 tokens, 4 adapters of rank 8, scale 2, token t on adapter
    t mod 5 where 4 is base only."""
    sites = [Site.fused(0, 1024, [("proj", 1024)])]
    slot = [(t % 5) + 1 if (t % 5) < 4 else 0 for t in range(16)]
    return Workload("plumbing-1024", sites, [8] * 4, 2.0, [1] * 16, slot, seed)


def config2(seed=0, tokens=64, adapters=16, rank=16, base_frac=0.25):
    """Decode mixed batch: hidden 4096 / intermediate 12288 block, 64 one-token sequences, 16 adapters of
    rank 16 on all seven projections, a quarter of the tokens base only."""
    sites = block_sites(4096, 12288, 1024)
    rng = np.random.default_rng([seed, 7])
    n_base = int(round(tokens * base_frac))
    slot = np.concatenate([np.zeros(n_base, np.int32), rng.integers(1, adapters + 1, tokens - n_base)])
    rng.shuffle(slot)
    return Workload("decode-4096x12288-64tok-16xr16", sites, [rank] * adapters, 2.0, [1] * tokens, slot, seed)


def config3(seed=0, seqs=8, seq_len=2048, rank=64):
    """Prefill segments: 8 sequences of 2048 tokens, one rank-64 adapter each, scale 1."""
    sites = block_sites(4096, 12288, 1024)
    return Workload(f"prefill-4096x12288-{seqs}x{seq_len}-r{rank}", sites, [rank] * seqs, 1.0, [seq_len] * seqs,
                    list(range(1, seqs + 1)), seed)


def config4(seed=0, tokens=256, adapters=128, two_part=False):
    """Heterogeneous ranks {8,16,32,64,128} over one 4096 -> 12288 layer, Zipf(1.1) popularity, 10% base."""
    mods = [("mlp.gate_proj", 12288), ("mlp.up_proj", 12288)] if two_part else [("mlp.gate_proj", 12288)]
    sites = [Site.fused(0, 4096, mods)]
    ranks = [[8, 16, 32, 64, 128][i % 5] for i in range(adapters)]
    rng = np.random.default_rng([seed, 9])
    n_base = int(round(tokens * 0.1))
    w = 1.0 / np.arange(1, adapters + 1) ** 1.1
    slot = np.concatenate([np.zeros(n_base, np.int32), rng.choice(adapters, tokens - n_base, p=w / w.sum()) + 1])
    rng.shuffle(slot)
    return Workload("hetero-4096x12288-256tok-128ad", sites, ranks, 1.0, [1] * tokens, slot.astype(np.int32), seed,
                    max_rank=128)


def config5(seed=0, adapters=32, rank=32, hidden=5120, inter=17408, q_width=6144, decode=256, chunks=(128, 128)):
    """27B-shaped layer (hidden 5120, intermediate 17408, q width 6144), 512 tokens = 256 one-token decode
    sequences first, then 2 prompt chunks of 128; 32 adapters of rank 32, uniform per sequence. The sites are
    the FULL layers; ``modes`` says how each is sharded in tensor-parallel mode (column-parallel q and
    gate/up, row-parallel o and down): see tp.shard_workload."""
    sites = [
        Site.fused(0, hidden, [("self_attn.q_proj", q_width)]),
        Site.fused(0, q_width, [("self_attn.o_proj", hidden)]),
        Site.fused(0, hidden, [("mlp.gate_proj", inter), ("mlp.up_proj", inter)]),
        Site.fused(0, inter, [("mlp.down_proj", hidden)]),
    ]
    rng = np.random.default_rng([seed, 11])
    row_n = [1] * decode + list(chunks)
    slot = rng.integers(1, adapters + 1, len(row_n))
    wl = Workload(f"tp-{hidden}x{inter}-{sum(row_n)}tok-{adapters}xr{rank}", sites, [rank] * adapters, 1.0, row_n, slot,
                  seed)
    wl.modes = ["column", "row", "column", "row"]
    return wl
