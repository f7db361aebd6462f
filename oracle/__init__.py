"""CPU oracle: a restatement of the reference's arithmetic for the projection / gated-delta-rule path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this; it is used by `tests/`, by the smoke
check and by the CPU-baseline leg of the benchmark as the checker / the timed CPU arm, never as a fallback.

Pinning status
  * gated delta rule: PINNED - reproduces the reference's self-contained known-answer tests
    (src/archs/qwen35_text.rs:1391-1462: closed-form inputs, in-test scalar recurrence, tolerance 1e-4), and the
    two independent forms here (token-sequential, 32-token chunked) agree with each other.
  * GeGLU elementwise: PINNED against the 16-value test of src/archs/modernbert.rs:743-766 (expected values
    from the exact-erf GELU definition the test itself uses).
  * RoPE: checked the way the reference's own test does (fused index arithmetic against the plain rotate-half on
    the test's formula inputs; that test holds no expected numbers); the f32 tables replay
    `rotary_tables_resolve_every_position` (src/archs/modernbert.rs:1359-1406).
  * RMSNorm: PINNED by replaying `rms_norm_matches_the_open_coded_reference` (src/archs/qwen35_text.rs:1214-1262,
    formula inputs, 1e-5 / 1e-2). LayerNorm: restated from the cited formula, cross-checked against torch.
  * Attention masks and softmax: PINNED by replaying the reference's known-answer tests
    (src/archs/modernbert.rs:1408-1443 mask values, :1506-1533 windowed == dense within 1e-5, :1536-1580 bf16
    softmax / mask finiteness).
  * Qwen3.5 decoder stack (oracle/qwen35.py) and ModernBERT encoder stack (oracle/modernbert.py): cross-checked
    against the `transformers` implementations of the same architectures on random-init weights (f32, 1e-5).
  * Linear / GEMM arithmetic: PARITY UNPINNED - the only reference tests that pin it are whole-model snapshots
    that need Hugging Face checkpoints which are not available offline, and the arithmetic itself lives in
    third-party crates (candle-core / candle-nn 0.11.0, gemm 0.19.0) whose source is not part of the reference
    tree. It is restated from the public contract `Linear::forward(x) = x Wᵀ (+ b)` with f32 accumulation.
"""
from .projection import (geglu, linear, mlp_modernbert, mlp_qwen35, round_bf16, swiglu)  # noqa: F401
from .delta_rule import (causal_conv_silu, chunked_delta_rule, delta_inputs, finish_delta, sequential_delta_rule)  # noqa: F401
from .norm import layer_norm, rms_norm, rope, rope_qkv_indexed, rope_qkv_test_inputs  # noqa: F401,E402
from .modernbert import (EncoderConfig, attention, attention_softmax, eager_attention, encoder_forward, encoder_layer,  # noqa: F401,E402
                         global_attention_mask, init_weights, local_attention_mask, windowed_attention)
from .qwen35 import DecoderConfig, causal_attention, decoder_forward, decoder_layer  # noqa: F401,E402
from . import qwen35  # noqa: F401,E402
from . import laya  # noqa: F401,E402
