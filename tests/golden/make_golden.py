"""Generates tests/golden/kat.npz: the reference's deterministic test fixtures evaluated exactly.

The reference stores no golden files; its correctness tests fill inputs with fixed integer
patterns and compare against loops (t2s/tests/correctness/util/util.h:52-65 new_data_2d
SEQUENTIAL = i+j+1, :100-114 new_data_3d SEQUENTIAL = i+j+k, :197-224 new_data_6D CONSTANT = 1;
t2s/tests/correctness/aot/gemm-run.cpp:50-59 ina(k,i) = k+i, inb(j,k) = j-k). Because those
patterns are small integers, the expected outputs are exact integers; this script computes them
in int64 with numpy (independently of oracle/oracle.cpp) and stores inputs and outputs.
Arrays are stored C-contiguous with numpy's LAST axis = Halide dimension 0.

Run from the repository root: python tests/golden/make_golden.py"""
import os

import numpy as np

out = {}

# --- AOT GEMM test (aot/gemm-run.cpp:35-61): TOTAL_I=16, TOTAL_J=32, TOTAL_K=2048
I, J, K = 16, 32, 2048
ina = (np.arange(K)[None, :] + np.arange(I)[:, None]).astype(np.int64)            # ina(k,i) = k + i -> [i][k]
inb = (np.arange(J)[None, :] - np.arange(K)[:, None]).astype(np.int64)            # inb(j,k) = j - k -> [k][j]
out["aot_gemm_a"] = ina.astype(np.float32)
out["aot_gemm_b"] = inb.astype(np.float32)
out["aot_gemm_c_exact"] = ina @ inb                                               # exact integers (|c| < 2^53)

# --- small SEQUENTIAL GEMM (util.h new_data_2d: b(i,j) = i + j + 1) as in correctness/gemm tests, 64^3
n = 64
a2 = (np.arange(n)[:, None] + np.arange(n)[None, :] + 1).astype(np.int64)
out["seq_gemm_a"] = a2.astype(np.float32)
out["seq_gemm_b"] = a2.astype(np.float32)
out["seq_gemm_c_exact"] = a2 @ a2

# --- TTM of buffer/tmm_small.cpp: L=I=J=K=8, a = new_data_3d SEQUENTIAL, b = new_data_2d SEQUENTIAL
L = I3 = J3 = K3 = 8
a3 = (np.arange(J3)[:, None, None] + np.arange(I3)[None, :, None] + np.arange(L)[None, None, :]).astype(np.int64)  # [j][i][l]
b3 = (np.arange(K3)[:, None] + np.arange(L)[None, :] + 1).astype(np.int64)                                         # [k][l]
out["seq_ttm_a"] = a3.astype(np.float32)
out["seq_ttm_b"] = b3.astype(np.float32)
out["seq_ttm_c_exact"] = np.einsum("jil,kl->kji", a3, b3)

# --- MTTKRP with the same generators (util.h:464-481 takes a(L,I,K), b(K,J), c(L,J))
a4 = (np.arange(8)[:, None, None] + np.arange(8)[None, :, None] + np.arange(8)[None, None, :]).astype(np.int64)    # [k][i][l]
b4 = (np.arange(8)[:, None] + np.arange(8)[None, :] + 1).astype(np.int64)                                          # [r][k]
c4 = (np.arange(8)[:, None] + np.arange(8)[None, :] + 1).astype(np.int64)                                          # [r][l]
out["seq_mttkrp_a"] = a4.astype(np.float32)
out["seq_mttkrp_b"] = b4.astype(np.float32)
out["seq_mttkrp_c"] = c4.astype(np.float32)
out["seq_mttkrp_d_exact"] = np.einsum("kil,rl,rk->ri", a4, c4, b4)

# --- CONSTANT = 1 conv (new_data CONSTANT): every output equals CI*KY*KX
out["const_conv_expected"] = np.array([16 * 3 * 3], np.int64)

np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "kat.npz"), **out)
print({k: v.shape for k, v in out.items()})
