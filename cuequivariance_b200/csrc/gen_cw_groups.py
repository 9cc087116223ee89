"""Generates ``generated/cw_groups.cuh``: straight-line arithmetic for channelwise tensor
products, one struct per *group* (all paths that read the same irrep of the first operand).

Why generated code: the Clebsch-Gordan tensors are sparse with a pattern known at build
time.  Written out as straight-line FMAs every accumulator and every operand stays in a
register (registers cannot be indexed dynamically), and no multiply is spent on a zero.

For a path (l1, l2, l3) with coupling tensor C[i, j, k] the kernels use, per edge,
    M[i, k] = sum_j C[i, j, k] * x2[j]                  (channel independent)
    forward : out[k, u] += w[u] * sum_i M[i, k] * x1[i, u]
    backward: S[i, u]   = sum_k M[i, k] * g[k, u]
              gx1[i, u] += w[u] * S[i, u];   gw[u] = sum_i S[i, u] * x1[i, u]
              gx2[j]    += sum_{i,k} C[i, j, k] * sum_u w[u] x1[i, u] g[k, u]
Only the non-zero (i, k) pairs appear.  The numeric value of every M entry is computed at
run time from a small term table (the kernel needs only the *pattern* at compile time), so
normalisation factors of the descriptor can change without regenerating anything.

    python cuequivariance_b200/csrc/gen_cw_groups.py        # rewrites generated/cw_groups.cuh
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import numpy as np  # noqa: E402

from cuequivariance_b200.channelwise import group_signature as _signature, pair_pattern, split_group, value_pattern  # noqa: E402

# Groups to build: (l1, [(l2, l3), ...]).  The list below is the family used by MACE-style
# models: second operand 0e+1o+..+L2 (spherical harmonics), outputs filtered to natural
# parity irreps up to L3.
FAMILIES = [(3, 3)]  # (L2, L3) : l1 ranges over 0..3


def group_paths(l1: int, L2: int, L3: int) -> list[tuple[int, int]]:
    """(l2, l3) of every path of the group, in the descriptor's path order (l2 ascending,
    then l3 ascending) with l1+l2+l3 even (natural parity in, natural parity out)."""
    out = []
    for l2 in range(L2 + 1):
        for l3 in range(abs(l1 - l2), min(l1 + l2, L3) + 1):
            if (l1 + l2 + l3) % 2 == 0:
                out.append((l2, l3))
    return out


def group_name(l1: int, paths) -> str:
    return f"CwGroup_l{l1}_" + "_".join(f"{a}{b}" for a, b in paths)


def group_signature(l1: int, paths) -> str:
    return _signature(l1, paths)


def emit_group(l1: int, paths) -> str:
    d1 = 2 * l1 + 1
    name = group_name(l1, paths)
    pats = [pair_pattern(l1, l2, l3, "k") for l2, l3 in paths]
    pats_i = [pair_pattern(l1, l2, l3, "i") for l2, l3 in paths]
    d3s = [2 * l3 + 1 for _, l3 in paths]
    d2s = [2 * l2 + 1 for l2, _ in paths]
    npair = [len(p) for p in pats]
    pair_off = np.concatenate([[0], np.cumsum(npair)]).tolist()
    out_off = np.concatenate([[0], np.cumsum(d3s)]).tolist()
    ptot = pair_off[-1]
    ptot_pad = (ptot + 3) // 4 * 4
    vals = [value_pattern(l1, l2, l3) for l2, l3 in paths]
    val_off = np.concatenate([[0], np.cumsum([len(v) for v, _ in vals])]).tolist()
    fwd_terms = sum(len(t) for v, _ in vals for t in v)
    L = []
    A = L.append
    A(f"struct {name} {{")
    A(f"  static constexpr int L1 = {l1};")
    A(f"  static constexpr int D1 = {d1};")
    A(f"  static constexpr int NPATH = {len(paths)};")
    A(f"  static constexpr int NPAIR = {ptot};")
    A(f"  static constexpr int NPAIR_PAD = {ptot_pad};")
    A(f"  static constexpr int NVAL = {val_off[-1]};      // distinct values among the M entries (forward table)")
    A(f"  static constexpr int NTERM_FWD = {fwd_terms};")
    A(f"  static constexpr int SUMD3 = {out_off[-1]};")
    A(f"  static constexpr int MAXD3 = {max(d3s)};")
    A(f"  static constexpr int NX2 = {max(l2 for l2, _ in paths) ** 2 + 2 * max(l2 for l2, _ in paths) + 1};")
    A("  static constexpr const char* signature() { return \"%s\"; }" % group_signature(l1, paths))
    A("  __host__ __device__ static constexpr int d3(int p) { constexpr int t[NPATH] = {%s}; return t[p]; }" % ", ".join(map(str, d3s)))
    A("  __host__ __device__ static constexpr int out_offset(int p) { constexpr int t[NPATH + 1] = {%s}; return t[p]; }" % ", ".join(map(str, out_off)))
    A("  __host__ __device__ static constexpr int pair_offset(int p) { constexpr int t[NPATH + 1] = {%s}; return t[p]; }" % ", ".join(map(str, pair_off)))

    # ---- forward ------------------------------------------------------------------------
    A("  // acc[out_offset(p) + k][c] += W[p][c] * sum_i (+-)V[slot(i,k)] * X[i][c];  V = the distinct values of M")
    A("  template <int P, int C>")
    A("  __device__ __forceinline__ static void fwd_path(const float (&X)[D1][C], const float (&W)[C], const float* __restrict__ M,")
    A("                                                  float (&acc)[SUMD3][C]) {")
    for p, (pat, d3) in enumerate(zip(pats, d3s)):
        A(f"    if constexpr (P == {p}) {{")
        # load the distinct values of this path as float4 where aligned
        values, vpairs = vals[p]
        A(f"      float m[{len(values)}];")
        A(f"      cw_load_m<{val_off[p]}, {len(values)}>(M, m);")
        by_i2: dict[int, list] = {}
        for (i, k, s, sign) in vpairs:
            by_i2.setdefault(i, []).append((("-" if sign < 0 else "") + f"m[{s}]", k))
        if d1 < d3:
            # fewer input than output components: scale the inputs by the weight once (d1 multiplies)
            # and add every product straight into its accumulator, instead of summing unweighted
            # products in temporaries and scaling d3 of them at the end
            A(f"      float xw[{d1}][C];")
            for i in sorted(by_i2):
                A(f"      CW_MULV4(xw[{i}], W, X[{i}]);")
            for i in sorted(by_i2):
                for q, k in by_i2[i]:
                    A(f"      CW_FMA4(acc[{out_off[p] + k}], {q}, xw[{i}]);")
        else:
            # i-major emission: consecutive multiply-adds go to different accumulators t[k], so that
            # the chains over i of the d3 outputs interleave instead of running one after the other
            A(f"      float t[{d3}][C];")
            seen_k = set()
            for i in sorted(by_i2):
                for q, k in by_i2[i]:
                    if k in seen_k:
                        A(f"      CW_FMA4(t[{k}], {q}, X[{i}]);")
                    else:
                        seen_k.add(k)
                        A(f"      CW_MUL4(t[{k}], {q}, X[{i}]);")
            for k in range(d3):
                if k in seen_k:
                    A(f"      CW_FMAV4(acc[{out_off[p] + k}], W, t[{k}]);")
        A("    }")
    A("  }")

    # ---- backward -----------------------------------------------------------------------
    A("  // per path, pairs ordered by i: S[i] = sum_k M[q] G[k];  gX[i] += W*S[i];  gw = sum_i S[i] X[i];")
    A("  //           r[j] += c * dot4(W*X[i], G[k]) over the non-zero (i, j, k)")
    A("  // NEED_R = false leaves the x2-gradient partials (and the products that only feed them) out")
    A("  template <int P, int C, bool NEED_R, class Coef>")
    A("  __device__ __forceinline__ static void bwd_path(const float (&X)[D1][C], const float (&W)[C], const float* __restrict__ M,")
    A("                                                  const float (&G)[MAXD3][C], const Coef& coef,")
    A("                                                  float (&gX)[D1][C], float (&gw)[C], float (&r)[16]) {")
    term_cursor = 0
    for p, (pat, d3, d2) in enumerate(zip(pats_i, d3s, d2s)):
        l2 = paths[p][0]
        j_base = l2 * l2  # offset of irrep l2 inside x2 = 0e+1o+2e+...
        A(f"    if constexpr (P == {p}) {{")
        q0 = pair_off[p]
        A("#pragma unroll")
        A("      for (int c = 0; c < C; ++c) gw[c] = 0.f;")
        by_i: dict[int, list] = {}
        for q, (i, k, terms) in enumerate(pat):
            by_i.setdefault(i, []).append((q, k, terms))
        # the x2 gradient needs sum_u w[u] x1[i,u] g[k,u]: the weight is folded into whichever of
        # the two factors has fewer components (d1 or d3 multiplies per path)
        scale_g = d3 < d1
        if scale_g:
            ks = sorted({k for lst in by_i.values() for _, k, _ in lst})
            A(f"      float gs[{d3}][C];")
            for k in ks:
                A(f"      CW_MULV4(gs[{k}], W, G[{k}]);")
        t = term_cursor
        for i in range(d1):
            lst = by_i.get(i, [])
            if not lst:
                continue
            qa = lst[0][0]
            A("      {")
            A(f"        float m[{len(lst)}];")
            A(f"        cw_load_m<{q0 + qa}, {len(lst)}>(M, m);")
            if scale_g:
                A("        float s[C];")
            else:
                A("        float s[C], xw[C];")
                A(f"        CW_MULV4(xw, W, X[{i}]);")
            for n, (q, k, terms) in enumerate(lst):
                if n == 0:
                    A(f"        CW_MUL4(s, m[{q - qa}], G[{k}]);")
                else:
                    A(f"        CW_FMA4(s, m[{q - qa}], G[{k}]);")
                if scale_g:
                    A(f"        if constexpr (NEED_R) {{ const float v = CW_DOT4(X[{i}], gs[{k}]);")
                else:
                    A(f"        if constexpr (NEED_R) {{ const float v = CW_DOT4(xw, G[{k}]);")
                for j, _c in terms:
                    A(f"          r[{j_base + j}] = fmaf(coef.c[{t}], v, r[{j_base + j}]);")
                    t += 1
                A("        }")
            A(f"        CW_FMAV4(gX[{i}], W, s);")
            A(f"        CW_FMAV4(gw, s, X[{i}]);")
            A("      }")
        term_cursor = t
        A("    }")
    A("  }")
    A(f"  static constexpr int NTERM = {term_cursor};")
    A("};")
    return "\n".join(L)


def all_groups():
    seen, out = set(), []
    for L2, L3 in FAMILIES:
        for l1 in range(4):
            paths = group_paths(l1, L2, L3)
            if not paths:
                continue
            for part in split_group(l1, paths):
                key = (l1, tuple(part))
                if key not in seen:
                    seen.add(key)
                    out.append((l1, part))
    return out


def main():
    groups = all_groups()
    parts = [
        "// GENERATED by gen_cw_groups.py - do not edit.  Straight-line Clebsch-Gordan arithmetic of the",
        "// channelwise tensor product, one struct per group of paths sharing an irrep of operand 1.",
        "#pragma once",
        '#include "../cw_macros.cuh"',
        "",
    ]
    for l1, paths in groups:
        parts.append(emit_group(l1, paths))
        parts.append("")
    names = [group_name(l1, p) for l1, p in groups]
    parts.append("#define CW_FOR_EACH_GROUP(X) \\")
    parts.append(" \\\n".join(f"  X({n})" for n in names))
    parts.append("")
    os.makedirs(os.path.join(HERE, "generated"), exist_ok=True)
    path = os.path.join(HERE, "generated", "cw_groups.cuh")
    text = "\n".join(parts)
    if not os.path.exists(path) or open(path).read() != text:
        open(path, "w").write(text)
    return [(group_signature(l1, p), n) for (l1, p), n in zip(groups, names)]


if __name__ == "__main__":
    for sig, n in main():
        print(sig, n)
