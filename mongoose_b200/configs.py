"""Model shapes for the fused decode engine.

The constructor arguments are the positional ints of the reference's
``NewCUDAFusedInference(eng, dim, kvDim, headDim, nHeads, nKVHeads, ffnDim,
vocabSize, nLayers, maxSeq, ropeTheta)`` (cuda_fused_infer.go:144), plus the
RMSNorm epsilon the reference hard-codes (kernels/mongoose.cu:170).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

# weight storage formats (values match include/mongoose_kernels.h MG_FMT_*)
FMT_Q8_0 = 0
FMT_Q4_0 = 1
FMT_F16 = 2

# slots of the reference's weight index scheme, idx = layer*12 + slot
# (cuda_fused_infer.go:241-272)
SLOT_NORM1, SLOT_WQ, SLOT_WK, SLOT_WV = 0, 1, 2, 3
SLOT_BQ, SLOT_BK, SLOT_BV = 4, 5, 6
SLOT_WO, SLOT_NORM2, SLOT_GATE, SLOT_UP, SLOT_DOWN = 7, 8, 9, 10, 11
MATRIX_SLOTS = (SLOT_WQ, SLOT_WK, SLOT_WV, SLOT_WO, SLOT_GATE, SLOT_UP, SLOT_DOWN)


@dataclass(frozen=True)
class ModelConfig:
    name: str
    dim: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_dim: int
    vocab: int
    n_layers: int
    max_seq: int
    rope_theta: float
    eps: float = 1e-6
    layer_fmt: int = FMT_Q8_0   # format of the seven per-layer matrices
    head_fmt: int = FMT_Q8_0    # format of lm_head (and of the tied embedding)

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def num_weights(self) -> int:
        """NumWeights() of the reference (cuda_fused_infer.go:231-233)."""
        return self.n_layers * 12 + 2

    def matrix_shape(self, slot: int) -> tuple[int, int]:
        """(rows, cols) = (out, in) of a per-layer matrix slot."""
        d, kv, f = self.dim, self.kv_dim, self.ffn_dim
        return {SLOT_WQ: (d, d), SLOT_WK: (kv, d), SLOT_WV: (kv, d), SLOT_WO: (d, d),
                SLOT_GATE: (f, d), SLOT_UP: (f, d), SLOT_DOWN: (d, f)}[slot]

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)


def fmt_row_bytes(fmt: int, cols: int) -> int:
    if fmt == FMT_Q8_0:
        return cols // 32 * 34
    if fmt == FMT_Q4_0:
        return cols // 32 * 18
    return cols * 2


def weight_bytes_per_token(cfg: ModelConfig) -> int:
    """Quantized bytes of the 7*L layer matrices plus lm_head: what one decode
    token must stream from HBM."""
    per_layer = sum(r * fmt_row_bytes(cfg.layer_fmt, c)
                    for r, c in (cfg.matrix_shape(s) for s in MATRIX_SLOTS))
    return per_layer * cfg.n_layers + cfg.vocab * fmt_row_bytes(cfg.head_fmt, cfg.dim)


def kv_bytes_per_position(cfg: ModelConfig) -> int:
    """fp16 K and V of every layer for one cached position."""
    return 2 * cfg.n_layers * cfg.kv_dim * 2


QWEN25_05B = ModelConfig("qwen2.5-0.5b", dim=896, n_heads=14, n_kv_heads=2, head_dim=64, ffn_dim=4864,
                         vocab=151936, n_layers=24, max_seq=232, rope_theta=1e6)
QWEN25_05B_Q4 = QWEN25_05B.with_(name="qwen2.5-0.5b-q4_0", layer_fmt=FMT_Q4_0, head_fmt=FMT_F16)
TINYLLAMA_11B = ModelConfig("tinyllama-1.1b", dim=2048, n_heads=32, n_kv_heads=4, head_dim=64, ffn_dim=5632,
                            vocab=32000, n_layers=22, max_seq=1024, rope_theta=1e4)
QWEN25_7B = ModelConfig("qwen2.5-7b-class", dim=3584, n_heads=28, n_kv_heads=4, head_dim=128, ffn_dim=18944,
                        vocab=152064, n_layers=28, max_seq=384, rope_theta=1e6)
# small shapes for CPU-side tests and the GPU smoke run
TINY = ModelConfig("tiny", dim=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn_dim=352, vocab=1000,
                   n_layers=2, max_seq=48, rope_theta=1e4)
TINY_Q4 = TINY.with_(name="tiny-q4_0", layer_fmt=FMT_Q4_0, head_fmt=FMT_F16)

CONFIGS = {c.name: c for c in (QWEN25_05B, QWEN25_05B_Q4, TINYLLAMA_11B, QWEN25_7B, TINY, TINY_Q4)}
