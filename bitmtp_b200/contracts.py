"""Shape registry and decoding contracts (CPU-only, imports neither torch nor the native library).

Mirrors `bonsai_sft.gpu.contracts` of the reference
(src/bonsai_sft/gpu/contracts.py:11-124): the same registered (M, N, K) tables
and validation helpers, so callers that pre-validate against the registry keep
working.  Two differences, both additive:
  * the B200 kernels take every 1 <= M <= 32, K % 128 == 0, N % 8 == 0, so
    `supports_native_shape` accepts shapes outside the tables (W = 2, the
    8192 -> 28672 stress layer, test sizes);
  * the public device scope admits compute capability (10, 0) for the 4B model.
"""
from __future__ import annotations

import math

def _projection_shapes(dim, heads, kv_heads, head_dim, ffn, vocab, *, unfused):
    """(N, K) of every packed projection of one backbone: fused q|k|v and gate|up, o, down, the tied head, the
    key/value projection on its own, and (where the reference also registers them) the unfused q and gate."""
    q, kv = heads * head_dim, kv_heads * head_dim
    shapes = {(kv, dim), (q + 2 * kv, dim), (2 * ffn, dim), (dim, q), (dim, ffn), (vocab, dim)}
    if unfused:
        shapes |= {(q, dim), (ffn, dim)}
    return frozenset(shapes)


_PADDED_VOCAB = 151936
_WIDE = tuple(range(4, 11)) + (12, 16, 17)          # verify widths of D4/D8 blocks plus the prompt-tail widths
Q1_M = frozenset((1,) + _WIDE)
BONSAI_17B_NK = _projection_shapes(2048, 16, 8, 128, 6144, _PADDED_VOCAB, unfused=True)
T2_4B_M = frozenset(m for m in Q1_M if m == 1 or m >= 8)
T2_4B_NK = _projection_shapes(2560, 32, 8, 128, 9728, _PADDED_VOCAB, unfused=False)
MAX_WIDTH = 32


_GEOMETRY_KEYS_GPU = ('dim', 'n_layers', 'n_heads', 'n_kv_heads', 'head_dim', 'ffn_dim', 'vocab_size')
_GEOMETRY_KEYS_HF = ('hidden_size', 'num_hidden_layers', 'num_attention_heads',
                     'num_key_value_heads', 'head_dim', 'intermediate_size', 'vocab_size')
_BACKBONES = {
    # (dim, layers, heads, kv heads, head_dim, ffn) -> admitted block sizes
    (2048, 28, 16, 8, 128, 6144): (4, 8),
    (2560, 36, 32, 8, 128, 9728): (8,),
}
# 151669 is the released vocabulary; 151936 is its padded size, which synthetic
# checkpoints use directly.
_VOCABS = (151669, 151936)


def validate_public_model_scope(config: dict, *, hf: bool = False, quant: str = "ternary",
                                quantize_embedding: bool = True) -> None:
    """Geometry / quantisation-format scope of the public CLI.

    Same acceptance rule and error text as the reference
    (src/bonsai_sft/gpu/contracts.py:23-62): Bonsai-1.7B T2 with D in {4, 8} or
    Bonsai-4B T2 with D = 8, tied embeddings, ternary g128 quantisation.  An HF
    config without block_size is read as D = 8.
    """
    if not isinstance(config, dict):
        raise ValueError('public release requires a JSON object model configuration')
    keys = _GEOMETRY_KEYS_HF if hf else _GEOMETRY_KEYS_GPU
    values = [config.get(k) for k in keys]
    blocks = ()
    if all(type(v) is int for v in values) and values[-1] in _VOCABS:
        blocks = _BACKBONES.get(tuple(values[:-1]), ())
    problems = []
    if not blocks:
        problems.append('model_geometry')
    block_size = config.get('block_size', 8 if hf else None)
    if type(block_size) is not int or block_size not in blocks:
        problems.append('block_size')
    if config.get('tie_word_embeddings') is not True:
        problems.append('tie_word_embeddings')
    if hf:
        quant_ok = quant == 'ternary' and bool(quantize_embedding)
    else:
        quant_ok = (config.get('kernel_kind') == 't2g128'
                    and config.get('quantize_embedding', True) is True)
    if not quant_ok:
        problems.append('quantization')
    if problems:
        raise ValueError(
            'public release supports only Bonsai 1.7B T2 D4/D8 or Bonsai 4B T2 D8 '
            '(including D8 SFT exports); unsupported configuration fields: ' + ', '.join(problems))


def validate_public_device_scope(config: dict, capability) -> None:
    """The reference admits the 4B model on SM90 only (contracts.py:65-69); this build's
    kernels are sm_100a, so (10, 0) is the admitted capability for every model."""
    if tuple(capability) != (10, 0):
        raise ValueError('bitmtp_b200 kernels are built for sm_100a (B200); '
                         f'device capability {tuple(capability)} is unsupported')


_ONE_BIT_KINDS = ("q1", "w1a16")          # the reference's 1-bit kernels: known names, not built here
_GRAPH_ROLES = frozenset(("ar", "verify", "draft", "draft_fp8", "draft_bf16"))


def _registered(m: int, n: int, k: int) -> bool:
    return any(m in widths and (n, k) in shapes
               for widths, shapes in ((Q1_M, BONSAI_17B_NK), (T2_4B_M, T2_4B_NK)))


def supports_kernel_shape(kind: str, m: int, n: int, k: int) -> bool:
    """Whether (M, N, K) is one of the reference's registered triples (contracts.py:72-81)."""
    if kind == "t2g128":
        return _registered(m, n, k)
    if kind not in _ONE_BIT_KINDS:
        raise ValueError(f"unknown kernel kind: {kind!r}")
    return False


def supports_native_shape(m: int, n: int, k: int) -> bool:
    """What libbitmtp_b200's GEMV accepts."""
    return 1 <= m <= MAX_WIDTH and n >= 8 and n % 8 == 0 and k >= 128 and k % 128 == 0


def _refuse_shape(kind: str, m: int, n: int, k: int):
    raise RuntimeError(f"unsupported {kind} kernel shape: M={m}, N={n}, K={k}")


def require_kernel_shape(kind: str, m: int, n: int, k: int) -> None:
    supports_kernel_shape(kind, m, n, k) or _refuse_shape(kind, m, n, k)


def require_native_shape(m: int, n: int, k: int) -> None:
    supports_native_shape(m, n, k) or _refuse_shape("t2g128", m, n, k)


def supports_layer_kernel_shape(kind: str, m: int, n: int, k: int) -> bool:
    """The reference's variable-width layer forward uses the 4B kernels at M = 1 only (contracts.py:89-98)."""
    four_b = kind == "t2g128" and (n, k) in T2_4B_NK
    return m == 1 if four_b else supports_kernel_shape(kind, m, n, k)


def validate_verification_options(rabv_margin: float, exact_m1_verify: bool = False) -> None:
    """Strict verification accepts a zero margin only (contracts.py:101-108); a margin that is not a
    number at all is refused with the same message."""
    try:
        zero = math.isfinite(rabv_margin) and not rabv_margin
    except (TypeError, ValueError):
        zero = False
    if not zero:
        raise ValueError("strict verifier requires rabv_margin=0; nonzero margins are unsupported")


def validate_native_verifier(use_fp8=False, use_q1=False, use_w1a16=False) -> None:
    """The verifier projects through the backbone's own packed head (contracts.py:111-114)."""
    if any((use_fp8, use_q1, use_w1a16)):
        raise ValueError("strict verification requires the native verifier projection")


def validate_graph_roles(roles, capability=None) -> None:
    """Role names a session may capture graphs for (contracts.py:117-124)."""
    strangers = sorted(set(roles) - _GRAPH_ROLES)
    if strangers:
        raise ValueError(f"unsupported strict graph roles: {strangers}")
    fp8_capable = capability is None or tuple(capability) >= (8, 9)
    if "draft_fp8" in roles and not fp8_capable:
        raise ValueError("FP8 draft projection is unsupported on this GPU; use draft_bf16 or native draft")
