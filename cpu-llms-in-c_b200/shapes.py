"""Projection sets of the benchmark configurations and their algorithmic work.

bytes(projection, M) = N*K/2 + N*(K/64)*4 + M*K*2 + M*N*2   (fused gate/up: two
weight terms, one x term, one output term); flops = 2*M*N*K (x2 for gate/up).
No credit for padding, re-reads or layout overhead.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Projection:
    name: str
    k: int          # input columns
    n: int          # output rows
    fused: bool = False  # gate/up pair with SiLU-gate epilogue
    group: str = ""      # projections with the same non-empty group share x and one launch


def _layer(hidden, q, kv, mlp):
    return (
        Projection("q", hidden, q, group="qkv"),
        Projection("k", hidden, kv, group="qkv"),
        Projection("v", hidden, kv, group="qkv"),
        Projection("o", q, hidden),
        Projection("gate_up", hidden, mlp, fused=True),
        Projection("down", mlp, hidden),
    )


LAYER_SMALL = _layer(1024, 2048, 512, 3072)
LAYER_27B = _layer(5120, 6144, 1024, 17408)


def weight_bytes(p: Projection) -> int:
    one = p.n * p.k // 2 + p.n * (p.k // 64) * 4
    return 2 * one if p.fused else one


def algorithmic_bytes(p: Projection, m: int) -> int:
    return weight_bytes(p) + m * p.k * 2 + m * p.n * 2


def algorithmic_flops(p: Projection, m: int) -> int:
    return (2 if p.fused else 1) * 2 * m * p.n * p.k


def layer_bytes(layer, m: int) -> int:
    return sum(algorithmic_bytes(p, m) for p in layer)


def layer_flops(layer, m: int) -> int:
    return sum(algorithmic_flops(p, m) for p in layer)
