"""Seeded synthetic models for the decode-path configurations.

The reference's published runs use public checkpoints that cannot be fetched
here; these generators stand in for them with the same shapes, block sizes
and an N(0, 0.02) weight distribution.  Everything is derived from
``numpy.random.default_rng`` seeds so that every consumer (engine, tests,
benchmark) sees identical tensors.
"""
from __future__ import annotations

import numpy as np

from . import configs as mc


def single_matvec_case(seed: int = 0, N: int = 4864, K: int = 896):
    """One Q8_0 dequant-matvec: int8 blocks uniform in [-127,127], fp16 block
    scales |N(0,1)|*0.02/127, x ~ N(0,1).  Returns (raw blocks uint8 [N, K/32*34], x)."""
    rng = np.random.default_rng(seed)
    nb = K // 32
    q = rng.integers(-127, 128, size=(N, nb, 32), dtype=np.int8)
    d = (np.abs(rng.standard_normal((N, nb))) * 0.02 / 127.0).astype(np.float16)
    x = rng.standard_normal(K).astype(np.float32)
    blocks = np.empty((N, nb, 34), np.uint8)
    blocks[:, :, :2] = d.view(np.uint8).reshape(N, nb, 2)
    blocks[:, :, 2:] = q.view(np.uint8)
    return blocks.reshape(N, nb * 34), x


def tensor_f32(seed: int, idx: int, rows: int, cols: int, std: float = 0.02) -> np.ndarray:
    """The fp32 matrix for weight slot ``idx`` of a random-init model."""
    rng = np.random.default_rng([seed, idx])
    w = rng.standard_normal((rows, cols), dtype=np.float32)
    w *= np.float32(std)
    return w


def model_slots(cfg: mc.ModelConfig):
    """Yield (idx, kind, rows, cols, fmt) for every weight slot that is set.
    kind is "norm" or "matrix"."""
    for l in range(cfg.n_layers):
        base = l * 12
        yield base + mc.SLOT_NORM1, "norm", 1, cfg.dim, None
        yield base + mc.SLOT_NORM2, "norm", 1, cfg.dim, None
        for s in mc.MATRIX_SLOTS:
            r, c = cfg.matrix_shape(s)
            yield base + s, "matrix", r, c, cfg.layer_fmt
    yield cfg.n_layers * 12, "norm", 1, cfg.dim, None
    yield cfg.n_layers * 12 + 1, "matrix", cfg.vocab, cfg.dim, cfg.head_fmt


def norm_vector(seed: int, idx: int, dim: int, jitter: float = 0.0) -> np.ndarray:
    """RMSNorm weights: ones (random-init), optionally perturbed so that a kernel
    which ignores the norm weight cannot pass a test."""
    if jitter == 0.0:
        return np.ones(dim, np.float32)
    rng = np.random.default_rng([seed, idx, 7])
    return (1.0 + jitter * rng.standard_normal(dim)).astype(np.float32)


def prompt_ids(seed: int, n: int, vocab: int) -> np.ndarray:
    rng = np.random.default_rng([seed, 1 << 20])
    return rng.integers(0, vocab, size=n, dtype=np.int64).astype(np.int32)


def load_engine(engine, cfg: mc.ModelConfig, seed: int = 0, jitter: float = 0.0, on_matrix=None) -> None:
    """SetWeight every slot of a random-init model.  ``on_matrix(idx, w, fmt)`` is
    called with each fp32 matrix before it is dropped (benchmarks use it to hand the
    same tensor to the CPU baseline)."""
    for idx, kind, rows, cols, fmt in model_slots(cfg):
        if kind == "norm":
            v = norm_vector(seed, idx, cols, jitter)
            engine.SetWeight(idx, v)
            if on_matrix is not None:
                on_matrix(idx, v, None)
            continue
        w = tensor_f32(seed, idx, rows, cols)
        engine.SetWeight(idx, w)
        if on_matrix is not None:
            on_matrix(idx, w, fmt)
        del w
