"""Seeded inputs for comparing the CPU oracle with the reference's own host
functions.  Shared by the generator of tests/golden/ref_host.npz and by
tests/test_oracle_vs_ref.py, so the recorded reference outputs and the oracle
see the same bytes.  Every array is a pure function of its arguments."""
import numpy as np

from moonshine_b200 import synth

REF_LATENT, REF_EXPERT_HIDDEN, REF_EXPERTS, REF_TOP_K, REF_Q8_COLUMNS = 3584, 3072, 896, 16, 7168


def key(case: int, part: int) -> int:
    return synth.stream_key(9000 + case, part)


def bf16_values() -> np.ndarray:
    """float32 inputs of the bf16 conversion: halfway cases either side of even and
    odd, subnormals, infinities, a NaN, and hashed bit patterns."""
    special = np.array([0x00000000, 0x80000000, 0x3F808000, 0x3F818000, 0x3F807FFF, 0x3F808001,
                        0x7F7FFFFF, 0x7F800000, 0xFF800000, 0x7FC00001, 0x00000001, 0x00008000,
                        0x00018000, 0x007FFFFF, 0x477FF000, 0xC2F6E979], np.uint32)
    hashed = (synth.hash64(key(0, 0), np.arange(4096, dtype=np.uint64)) >> np.uint64(32)).astype(np.uint32)
    hashed = hashed[(hashed & 0x7F800000) != 0x7F800000]          # finite only
    return np.concatenate([special, hashed]).view(np.float32)


def activations(case: int, count: int, sigma: float = 1.0) -> np.ndarray:
    return synth.bf16_bits(synth.normal_f32(key(case, 1), count, sigma))


def bf16_matrix(case: int, rows: int, columns: int, sigma: float) -> np.ndarray:
    return synth.bf16_bits(synth.normal_f32(key(case, 2), rows * columns, sigma)).reshape(rows, columns)


def mxfp4_matrix(case: int, rows: int, columns: int, scale_low: int, scale_span: int, part: int = 3):
    packed = synth.bytes_uniform(key(case, part), rows * columns // 2).reshape(rows, columns // 2)
    scales = synth.bytes_uniform(key(case, part + 1), rows * columns // 32, scale_low, scale_span
                                 ).reshape(rows, columns // 32)
    return packed, scales


def router_rows(case: int, rows: int):
    """Logit rows of 896 with a bias; odd rows carry exact ties (logits and bias of
    expert 2j+1 copied from expert 2j for 40 pairs)."""
    logits = synth.uniform_f32(key(case, 5), rows * REF_EXPERTS, -4.0, 4.0).reshape(rows, REF_EXPERTS).copy()
    bias = synth.uniform_f32(key(case, 6), REF_EXPERTS, -0.15, 0.15).copy()
    tied_bias = bias.copy()
    for j in range(40):
        tied_bias[2 * j + 1] = tied_bias[2 * j]
        logits[1::2, 2 * j + 1] = logits[1::2, 2 * j]
    return logits, bias, tied_bias


def q8_rows(case: int, rows: int):
    q = synth.int8_uniform(key(case, 7), rows * REF_Q8_COLUMNS).reshape(rows, REF_Q8_COLUMNS)
    s = synth.uniform_f32(key(case, 8), rows * REF_Q8_COLUMNS // 128, 1e-4, 1e-3).reshape(rows, -1)
    return q, s


def expert_span(case: int, rank: int):
    """Six tensors of one expert at the reference's real shape, checkpoint order:
    w1.packed, w1.scale, w2.packed, w2.scale, w3.packed, w3.scale."""
    w1 = mxfp4_matrix(case, REF_EXPERT_HIDDEN, REF_LATENT, 119, 5, 10 + 10 * rank)
    w2 = mxfp4_matrix(case, REF_LATENT, REF_EXPERT_HIDDEN, 119, 5, 12 + 10 * rank)
    w3 = mxfp4_matrix(case, REF_EXPERT_HIDDEN, REF_LATENT, 119, 5, 14 + 10 * rank)
    return (*w1, *w2, *w3)
