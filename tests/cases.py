"""Case lists for the attention parity tests.

The shapes and option combinations are the coverage the reference's own GPU
suites pin (they are facts about coverage, re-expressed here as data):
  - SDPA_OPTIONS: packages/runntime/test/core/kernels/attention/checkSdpa.ts:34-52
  - PREFILL_SHAPES: attn.gpu.test.ts:49-266 and attnFlash.gpu.test.ts:20-117
  - DECODE_CASES: attnDecode.gpu.test.ts:38-91 (+ the 72-head split case the
    reference marks as a known bug, :93-99, which must be correct here)
  - ZOO_SHAPES: packages/runntime/bench/kernels/attention.ab.ts:127-294
"""
from __future__ import annotations

import math

from oracle import SdpaCase

INF = math.inf

# (name, overrides) — every mask and input form, for a square self-attention
# shape with 4 query heads and 2 kv heads.
SDPA_OPTIONS = [
    ("full", {}),
    ("causal", dict(windowRight=0)),
    ("sliding", dict(windowLeft=3, windowRight=0)),
    ("two_sided", dict(windowLeft=2, windowRight=1)),
    ("sinks", dict(sinks=True, windowRight=0)),
    ("segments", dict(segments=True)),
    ("segments_causal", dict(segments=True, windowRight=0)),
    ("packed", dict(packed=True, windowRight=0)),
    ("packed_sinks_segments", dict(packed=True, sinks=True, segments=True)),
    ("keybias", dict(keyBias=True, windowRight=0)),
    ("keybias_sinks_segments", dict(keyBias=True, sinks=True, segments=True)),
    ("gqa_4to1", dict(kvHeads=1, windowRight=0)),
    ("gqa_3to1", dict(qHeads=6, kvHeads=2, sinks=True, windowRight=0)),
    ("mha", dict(kvHeads=4)),
]


def option_cases(t: int, headDim: int):
    base = SdpaCase(qLen=t, kvLen=t, qHeads=4, kvHeads=2, headDim=headDim)
    return [(f"{name}-t{t}-hd{headDim}", base.with_(**o)) for name, o in SDPA_OPTIONS]


def _c(**kw) -> SdpaCase:
    return SdpaCase(**kw)


# Edge shapes from the row-kernel and flash suites.
PREFILL_SHAPES = [
    ("hd1", _c(qLen=5, kvLen=5, qHeads=2, kvHeads=1, headDim=1)),
    ("hd200_causal", _c(qLen=9, kvLen=9, qHeads=2, kvHeads=2, headDim=200, windowRight=0)),
    ("cross_1700_keys", _c(qLen=5, kvLen=1700, qHeads=2, kvHeads=1, headDim=8)),
    ("qposoffset_small", _c(qLen=6, kvLen=20, qHeads=2, kvHeads=1, headDim=8, windowRight=0,
                            qPosOffset=14)),
    ("empty_rows_sinks_small", _c(qLen=6, kvLen=4, qHeads=2, kvHeads=1, headDim=8, windowLeft=0,
                                  sinks=True)),
    ("empty_rows_sinks_120", _c(qLen=120, kvLen=100, qHeads=2, kvHeads=1, headDim=8,
                                windowLeft=0, sinks=True)),
    ("keys_96", _c(qLen=96, kvLen=96, qHeads=2, kvHeads=1, headDim=8, windowRight=0)),
    ("keys_97", _c(qLen=97, kvLen=97, qHeads=2, kvHeads=1, headDim=8, windowRight=0)),
    ("segments_maxseg_90", _c(qLen=180, kvLen=180, qHeads=2, kvHeads=1, headDim=8, segments=True,
                              maxSegment=90)),
    ("segments_maxseg_100", _c(qLen=200, kvLen=200, qHeads=2, kvHeads=1, headDim=8,
                               segments=True, maxSegment=100)),
    ("hd512_causal", _c(qLen=7, kvLen=7, qHeads=1, kvHeads=1, headDim=512, windowRight=0)),
    ("rows_70000_keys_8", _c(qLen=70000, kvLen=8, qHeads=1, kvHeads=1, headDim=4)),
    ("rows_66000_keys_100", _c(qLen=66000, kvLen=100, qHeads=1, kvHeads=1, headDim=4)),
    ("rows_20000_window_2", _c(qLen=20000, kvLen=20000, qHeads=1, kvHeads=1, headDim=126,
                               windowLeft=2, windowRight=0)),
    ("every_option_long", _c(qLen=2097122, kvLen=2097122, qHeads=2, kvHeads=1, headDim=1,
                             windowLeft=2, windowRight=0, sinks=True, segments=True,
                             keyBias=True)),
    # flash-suite shapes
    ("cross_20x1000", _c(qLen=20, kvLen=1000, qHeads=2, kvHeads=1, headDim=32)),
    ("qposoffset_50", _c(qLen=20, kvLen=70, qHeads=2, kvHeads=1, headDim=32, windowRight=0,
                         qPosOffset=50)),
    ("window_40", _c(qLen=100, kvLen=100, qHeads=2, kvHeads=1, headDim=64, windowLeft=40,
                     windowRight=0)),
    ("empty_rows_sinks_40x20", _c(qLen=40, kvLen=20, qHeads=2, kvHeads=1, headDim=16,
                                  windowLeft=0, sinks=True)),
    ("segments_maxseg_32", _c(qLen=64, kvLen=64, qHeads=2, kvHeads=1, headDim=16, segments=True,
                              maxSegment=32)),
    ("no_subgroup_100", _c(qLen=100, kvLen=100, qHeads=2, kvHeads=1, headDim=64)),
]

FLASH_HEAD_DIMS = [16, 32, 48, 64, 128, 256, 512]
FLASH_SIZES = [("odd", 37, 37), ("one_tile", 16, 16), ("tile_plus_1", 17, 17), ("two_rows", 2, 2)]


def flash_cases():
    out = []
    for hd in FLASH_HEAD_DIMS:
        for name, ql, kl in FLASH_SIZES:
            out.append((f"hd{hd}-{name}", _c(qLen=ql, kvLen=kl, qHeads=2, kvHeads=1, headDim=hd,
                                             windowRight=0)))
    return out


def decode(kvLen: int, **kw) -> SdpaCase:
    """Decode as a model runs it: one query at the end of the cache."""
    base = dict(qLen=1, kvLen=kvLen, qHeads=4, kvHeads=2, headDim=16, windowRight=0,
                qPosOffset=kvLen - 1)
    base.update(kw)
    return SdpaCase(**base)


DECODE_CASES = [
    ("kv1", decode(1)),
    ("kv7", decode(7)),
    ("kv64", decode(64)),
    ("kv65", decode(65)),
    ("kv256", decode(256)),
    ("hd1", decode(40, headDim=1)),
    ("hd37", decode(40, headDim=37)),
    ("hd128", decode(40, headDim=128)),
    ("window10", decode(200, windowLeft=10)),
    ("sinks", decode(200, sinks=True)),
    ("gqa_to1", decode(50, kvHeads=1)),
    ("heads72", decode(50, qHeads=72, kvHeads=8)),
    ("full_not_at_end", decode(50, windowRight=INF, qPosOffset=10)),
    ("no_key_sinks", decode(5, windowLeft=0, windowRight=INF, qPosOffset=9, sinks=True)),
    ("kv257", decode(257)),
    ("kv2048", decode(2048)),
    ("kv5000", decode(5000)),
    ("kv600_hd37", decode(600, headDim=37)),
    ("kv600_hd128", decode(600, headDim=128)),
    ("kv1000_window10", decode(1000, windowLeft=10)),
    ("kv1000_sinks", decode(1000, sinks=True)),
    ("kv600_gqa_to1", decode(600, kvHeads=1)),
    ("kv600_heads64", decode(600, qHeads=64, kvHeads=8)),
    ("kv600_heads72", decode(600, qHeads=72, kvHeads=8)),
    ("kv300_no_key_sinks", decode(300, windowLeft=0, windowRight=INF, qPosOffset=400,
                                  sinks=True)),
]

# Row counts past the reference's grid limits (4,194,240 row-heads per 1-D
# grid, 2^24 for exact f32 counting, 65535 x 16 flash rows — the last one is a
# known bug there and must be correct here).
LARGE_ROW_CASES = [
    ("rows_past_grid_stride", _c(qLen=4194245, kvLen=4, qHeads=1, kvHeads=1, headDim=2)),
    ("rows_past_2p24", _c(qLen=2 ** 24 + 3, kvLen=2, qHeads=1, kvHeads=1, headDim=1)),
    ("rows_past_flash_grid", _c(qLen=65535 * 16 + 1, kvLen=4, qHeads=1, kvHeads=1, headDim=16)),
]

# One case per dispatch route of the reference, with the zoo models' shapes.
ZOO_SHAPES = [
    ("moonshine_tiny_self_decode", "f32", _c(qLen=1, kvLen=120, qHeads=8, kvHeads=8, headDim=36,
                                             windowRight=0, qPosOffset=119)),
    ("decode_256_hd64", "f16", _c(qLen=1, kvLen=256, qHeads=8, kvHeads=8, headDim=64,
                                  windowRight=0, qPosOffset=255)),
    ("decode_hd37_full", "f32", _c(qLen=1, kvLen=64, qHeads=4, kvHeads=4, headDim=37)),
    ("moonshine_tiny_cross_1500", "f32", _c(qLen=1, kvLen=1500, qHeads=8, kvHeads=8,
                                            headDim=36)),
    ("decode_gqa_2048", "f16", _c(qLen=1, kvLen=2048, qHeads=14, kvHeads=2, headDim=64)),
    ("privacy_filter", "f32", _c(qLen=512, kvLen=512, qHeads=14, kvHeads=2, headDim=64,
                                 windowLeft=128, windowRight=128, sinks=True)),
    ("streaming_encoder", "f16", _c(qLen=256, kvLen=256, qHeads=8, kvHeads=8, headDim=64,
                                    windowRight=0)),
    ("hd48_full", "f32", _c(qLen=128, kvLen=128, qHeads=6, kvHeads=6, headDim=48)),
    ("reverb_keybias", "f16", _c(qLen=335, kvLen=640, qHeads=12, kvHeads=6, headDim=128,
                                 keyBias=True)),
    ("gqa_causal_256", "f32", _c(qLen=256, kvLen=256, qHeads=16, kvHeads=4, headDim=64,
                                 windowRight=0)),
    ("embeddinggemma_sliding", "f16", _c(qLen=512, kvLen=512, qHeads=4, kvHeads=2, headDim=256,
                                         windowLeft=512, windowRight=512)),
    ("embeddinggemma_full", "f32", _c(qLen=512, kvLen=512, qHeads=4, kvHeads=1, headDim=512)),
    ("minilm_bucket_128", "f32", _c(qLen=128, kvLen=128, qHeads=12, kvHeads=12, headDim=32,
                                    packed=True, segments=True)),
    ("minilm_bucket_512", "f16", _c(qLen=512, kvLen=512, qHeads=12, kvHeads=12, headDim=32,
                                    packed=True, segments=True)),
    ("moonshine_tiny_encoder", "f32", _c(qLen=200, kvLen=200, qHeads=8, kvHeads=8, headDim=36)),
    ("moonshine_base_encoder", "f32", _c(qLen=200, kvLen=200, qHeads=8, kvHeads=8, headDim=52)),
    ("moonshine_tiny_encoder_f16", "f16", _c(qLen=200, kvLen=200, qHeads=8, kvHeads=8,
                                             headDim=36)),
    ("reverb_keybias_f32", "f32", _c(qLen=335, kvLen=640, qHeads=12, kvHeads=6, headDim=128,
                                     keyBias=True)),
    ("grid_limit_shape", "f16", _c(qLen=65536, kvLen=16, qHeads=64, kvHeads=1, headDim=8)),
]
