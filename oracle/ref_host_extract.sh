#!/bin/sh
# Cuts the reference's host-side checking functions out of its test programs
# into oracle/_ref/*.inc (git-ignored; see ref_host_wrap.cpp for what each range
# holds).  usage: ref_host_extract.sh <reference tree> <output directory>
set -eu
REF="$1"
OUT="$2"
mkdir -p "$OUT"
cut_range() {  # file first last name
    sed -n "$2,$3p" "$REF/tests/$1" > "$OUT/$4"
    test -s "$OUT/$4"
}
cut_range test_k3_moe_smoke.cu 35 46 smoke_enum.inc
cut_range test_k3_moe_smoke.cu 80 253 smoke_host.inc
cut_range test_k3_moe_smoke.cu 601 613 smoke_expert.inc
cut_range test_k3_q8_projection.cu 31 38 q8_enum.inc
cut_range test_k3_q8_projection.cu 50 76 q8_row.inc
cut_range test_k3_mxfp4_envelope.cu 114 130 env_decode.inc
cut_range test_k3_mxfp4_envelope.cu 265 278 env_f64.inc
# the ranges are line numbers of one revision of the tree: refuse any other
grep -q 'static inline float bf16_to_float' "$OUT/smoke_host.inc"
tail -n 1 "$OUT/smoke_host.inc" | grep -q '^}$'
head -n 1 "$OUT/smoke_expert.inc" | grep -q 'reference_mxfp4_gemv(cpu_expert_gate'
head -n 1 "$OUT/q8_row.inc" | grep -q 'q8_reference_row'
head -n 1 "$OUT/env_f64.inc" | grep -q 'double reference = 0.0;'
