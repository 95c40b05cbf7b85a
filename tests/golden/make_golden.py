"""Generates the committed fixtures of tests/golden/ from the CPU oracle.

The reference (MoYe.jl) is Julia and cannot be run where these tests run, so the fixtures are
outputs of the oracle restatement (oracle/), which is itself pinned to the reference's own
golden vectors by tests/test_oracle_layout.py and tests/test_oracle_host.py.  They freeze the
oracle's answers on the seeded inputs of the CPU-runnable configuration (fp32 256^3 host
gemm!, layout algebra on shape (8,(4,2),16) with random strides), so a later change of the
oracle or of the generators cannot silently move the target.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import host_oracle as ho  # noqa: E402
import layout_oracle as lo  # noqa: E402


def tup(x):
    if isinstance(x, tuple):
        return [tup(e) for e in x]
    return int(x)


def layout_cases():
    """Shape (8,(4,2),16) with (i) a random compact order and (ii) arbitrary strides in [0,4096]."""
    rs = np.random.Generator(np.random.PCG64(20261125))
    shape = (8, (4, 2), 16)
    cases = []
    for trial in range(6):
        if trial % 2 == 0:
            order = [int(v) for v in rs.permutation(4)]
            stride = lo.compact_order(lo.static(shape), lo.static((order[0], (order[1], order[2]), order[3])))
            stride = lo.dynamic(stride)
        else:
            v = [int(x) for x in rs.integers(0, 4097, size=4)]
            stride = (v[0], (v[1], v[2]), v[3])
        L = lo.SL(shape, stride)
        entry = {"shape": tup(shape), "stride": tup(stride)}
        entry["values"] = [int(L(i)) for i in range(1, 1025)]
        c = lo.coalesce(L)
        entry["coalesce"] = {"shape": tup(c.shape), "stride": tup(c.stride)}
        rhs = lo.SL((32, 2), (2, 64))
        comp = lo.composition(L, rhs)
        entry["composition_rhs"] = {"shape": [32, 2], "stride": [2, 64]}
        entry["composition"] = {"shape": tup(comp.shape), "stride": tup(comp.stride),
                                "values": [int(comp(i)) for i in range(1, int(lo.size(comp)) + 1)]}
        # logical_divide needs static strides with a well-defined complement: divide per mode by ints
        div = lo.logical_divide(L, (lo.SL(2), lo.SL(4), lo.SL(4)))
        entry["logical_divide_tile"] = [2, 4, 4]
        entry["logical_divide"] = {"shape": tup(div.shape), "stride": tup(div.stride),
                                   "values": [int(div(i)) for i in range(1, 1025)]}
        cases.append(entry)
    return cases


def main():
    ho.build()
    with open(os.path.join(HERE, "cfg1_layouts.json"), "w") as f:
        json.dump({"cases": layout_cases()}, f, separators=(",", ":"))
    # host gemm!: A (M,K), B (N,K), C (M,N) column-major fp32, U[-1,1) seeds 0/1
    M = N = K = 256
    A, B = ho.uniform_pm1(0, (M * K,)), ho.uniform_pm1(1, (N * K,))
    C = ho.matmul_kernel_f32(A, B, M, N, K, bM=128, bN=128, bK=8, tA=(32, 8), tC=(16, 16), use_tower=True)
    np.savez_compressed(os.path.join(HERE, "cfg1_host_gemm_f32_256.npz"), C=C.reshape(N, M).T)
    # small quantised / half goldens: raw operand bits + widened host result
    m, n, k = 64, 48, 128
    out = {}
    a16, b16 = ho.uniform_pm1_f16_bits(3, (m * k,)), ho.uniform_pm1_f16_bits(4, (n * k,))
    out["f16_a"], out["f16_b"] = a16, b16
    out["f16_c"] = ho.gemm_samples(a16, b16, ho.F16, m, n, k, np.arange(m, dtype=np.int32))
    a8, b8 = ho.uniform_s8(5, (m * k,)), ho.uniform_s8(6, (n * k,))
    out["s8_a"], out["s8_b"] = a8, b8
    out["s8_c"] = ho.gemm_samples(a8, b8, ho.S8, m, n, k, np.arange(m, dtype=np.int32))
    ae, be = ho.normal_e4m3_bits(7, (m * k,)), ho.normal_e4m3_bits(8, (n * k,))
    out["e4m3_a"], out["e4m3_b"] = ae, be
    out["e4m3_c"] = ho.gemm_samples(ae, be, ho.E4M3, m, n, k, np.arange(m, dtype=np.int32))
    ab, bb = ho.normal_bf16_bits(9, (16 * k,), 0.02), ho.normal_bf16_bits(10, (n * k,), 0.02)
    out["bf16_a"], out["bf16_b"] = ab, bb
    out["bf16_c"] = ho.gemm_samples(ab, bb, ho.BF16, 16, n, k, np.arange(16, dtype=np.int32))
    np.savez_compressed(os.path.join(HERE, "small_gemm_goldens.npz"), **out)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
