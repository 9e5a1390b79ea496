"""The handful of environment knobs the coded-projection path keeps.

The reference has a 24-variable registry spanning five ownership layers
(escha_mlx/envs.py); most of it selects between Metal kernel variants or
configures parts of the runtime this package does not contain.  What survives
here are the knobs that change what THIS path computes or which of its two
kernel families runs.  Names and parsing rules follow the reference so an
existing deployment's environment keeps its meaning.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Generic, TypeVar

T = TypeVar("T")


@dataclass(frozen=True)
class EnvVar(Generic[T]):
    name: str
    parser: Callable[[str], T]
    description: str
    default: T | None = None
    value_help: str = "a valid value"

    def is_set(self) -> bool:
        return self.name in os.environ

    def get(self, default: T | None = None) -> T | None:
        raw = os.environ.get(self.name)
        if raw is None or not raw.strip():
            return self.default if default is None else default
        try:
            return self.parser(raw)
        except (TypeError, ValueError) as exc:
            raise ValueError(f"{self.name} must be {self.value_help}, got {raw!r}") from exc


def _bool(value: str) -> bool:
    v = value.strip().lower()
    if v in {"1", "true", "yes", "on"}:
        return True
    if v in {"0", "false", "no", "off"}:
        return False
    raise ValueError("invalid boolean")


def _choice(*choices: str) -> Callable[[str], str]:
    allowed = frozenset(choices)

    def parse(value: str) -> str:
        v = value.strip().lower()
        if v not in allowed:
            raise ValueError("invalid choice")
        return v

    return parse


def _positive_int(value: str) -> int:
    parsed = int(value)
    if parsed < 1:
        raise ValueError("not positive")
    return parsed


def _split_k(value: str):
    v = value.strip().lower()
    return "auto" if v == "auto" else _positive_int(v)


ESCHA_MLX_BIAS = EnvVar(
    "ESCHA_MLX_BIAS", _bool, "apply the per-linear additive correction a dense export ships "
    "(default off, as the reference: escha_mlx/dense.py:107-132)", False, "a boolean")

ESCHA_MLX_LUT = EnvVar(
    "ESCHA_MLX_LUT", _bool, "decode through the 65,536-entry fp16 table instead of the integer "
    "hash (bit-identical; honoured by decode_tiles and the reference-order GEMV)", False,
    "a boolean")

ESCHA_MLX_FUSED_HAD = EnvVar(
    "ESCHA_MLX_FUSED_HAD", _bool, "fuse the output Hadamard/rout transform into the GEMV "
    "epilogue (bit-identical to the separate transform kernel)", True, "a boolean")

ESCHA_MLX_SPLITK = EnvVar(
    "ESCHA_MLX_SPLITK", _split_k, "split factor of the input dimension: an integer pins it, "
    "'auto' uses the grid-filling policy", "auto", "'auto' or a positive integer")

ESCHA_MLX_GEMV = EnvVar(
    "ESCHA_MLX_GEMV", _choice("mma", "reforder"), "GEMV kernel family: 'mma' = tensor-core "
    "kernel (default), 'reforder' = scalar kernel in the reference kernels' exact accumulation "
    "order (bit-identical to them; slow)", "mma", "'mma' or 'reforder'")

ESCHA_MLX_DENSE_BLOCK_R = EnvVar(
    "ESCHA_MLX_DENSE_BLOCK_R", _positive_int, "pin rows-per-decode reported by "
    "msl.dense_block_r (the tensor-core kernel always shares a decode across 8 or 16 rows)",
    None, "a positive integer")

ESCHA_MLX_BLOCK_R = EnvVar(
    "ESCHA_MLX_BLOCK_R", _positive_int, "pin rows-per-group reported by "
    "EschaSparseMoeBlock._blocked_R", None, "a positive integer")


def registered() -> list[EnvVar]:
    return [v for v in globals().values() if isinstance(v, EnvVar)]


def validate_environment() -> None:
    """Parse every registered variable once so a malformed value fails early."""
    for var in registered():
        var.get()
