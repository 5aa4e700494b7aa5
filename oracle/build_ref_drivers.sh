#!/bin/bash
# Compiles the reference's UNMODIFIED host drivers, where they lie in the mounted reference tree,
#  (1) against the CPU oracle exposed under the interface symbols -> oracle/_ref/pin_*   (pins the oracle)
#  (2) against the per-design stubs + libt2sp_b200.so            -> tests/_bin/*         (GPU acceptance tests)
# No reference source is copied; only binaries are written, and both output folders are git-ignored.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
ROOT="$(dirname "$HERE")"
REF="${T2SP_REFERENCE:-/root/reference}"
PERF="$REF/t2s/tests/performance"
HAL="$REF/Halide/src/runtime"
CXX="${CXX:-g++}"
FLAGS="-O2 -std=c++17 -w -I $ROOT/include -I $HAL -I $REF/t2s/src"
mkdir -p "$HERE/_ref" "$ROOT/tests/_bin"
[ -d "$PERF" ] || { echo "reference tree not mounted at $REF"; exit 0; }

ORACLE_SRC="$HERE/oracle.cpp"
OFLAGS="-O3 -march=x86-64-v3 -ffp-contract=off -pthread"

# (1) oracle pins, CPU only
$CXX $FLAGS $OFLAGS -DTINY -DREF_GEMM    -I $PERF/gemm    $PERF/gemm/gemm-run-fpga.cpp       $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_gemm_tiny
$CXX $FLAGS $OFLAGS -DTINY -DREF_CONV    -I $PERF/conv    $PERF/conv/conv-run-fpga.cpp       $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_conv_tiny
$CXX $FLAGS $OFLAGS -DTINY -DREF_CAPSULE -I $PERF/capsule $PERF/capsule/capsule-run-fpga.cpp $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_capsule_tiny
$CXX $FLAGS $OFLAGS -DREF_AOT_GEMM $REF/t2s/tests/correctness/aot/gemm-run.cpp $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_aot_gemm
$CXX $FLAGS $OFLAGS -DTINY -DREF_SYRK -I $PERF/syrk $PERF/syrk/syrk-run-fpga.cpp $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_syrk_tiny
$CXX $FLAGS $OFLAGS -DTINY -DREF_GER -I $PERF/ger $PERF/ger/ger-run-fpga.cpp $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_ger_tiny
ONEC="$REF/t2s/tests/correctness/oneapi-integration"
$CXX -I $HERE/pin_include $FLAGS $OFLAGS -DTINY -DFPGA_EMULATOR -DREF_ONEAPI_CONV    -I $ONEC $ONEC/oneapi-target-5-run.cpp $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_oneapi_conv_tiny
$CXX -I $HERE/pin_include $FLAGS $OFLAGS -DTINY -DFPGA_EMULATOR -DREF_ONEAPI_CAPSULE -I $ONEC $ONEC/oneapi-target-6-run.cpp $HERE/ref_interface.cpp $ORACLE_SRC -o $HERE/_ref/pin_oneapi_capsule_tiny
# TTM and MTTKRP: the golden loops of the reference's test helper (correctness/util/util.h), compiled with
# a stand-in for the compiler's umbrella header (pin_include/Halide.h), against the oracle's restatements
UTIL="$REF/t2s/tests/correctness/util"
$CXX -I $HERE/pin_include $FLAGS $OFLAGS -I $UTIL $HERE/pin_contractions.cpp $ORACLE_SRC -o $HERE/_ref/pin_contractions

# (2) the same drivers against the product
LINK="-L $ROOT/t2sp_b200 -lt2sp_b200 -Wl,-rpath,\$ORIGIN/../../t2sp_b200"
STUBS="$ROOT/t2sp_b200/csrc/stubs"
if [ -f "$ROOT/t2sp_b200/libt2sp_b200.so" ]; then
  $CXX $FLAGS -DTINY -I $PERF/gemm    $PERF/gemm/gemm-run-fpga.cpp       $STUBS/gemm-interface.cpp    $LINK -o $ROOT/tests/_bin/gemm_tiny
  $CXX $FLAGS -DTINY -I $PERF/conv    $PERF/conv/conv-run-fpga.cpp       $STUBS/conv-interface.cpp    $LINK -o $ROOT/tests/_bin/conv_tiny
  $CXX $FLAGS -DTINY -I $PERF/capsule $PERF/capsule/capsule-run-fpga.cpp $STUBS/capsule-interface.cpp $LINK -o $ROOT/tests/_bin/capsule_tiny
  $CXX $FLAGS $REF/t2s/tests/correctness/aot/gemm-run.cpp $STUBS/host.cpp $LINK -o $ROOT/tests/_bin/aot_gemm
  # the oneAPI-flavoured GEMM driver (extra selector argument, returns the kernel time)
  ONE="$PERF/oneapi/src"
  $CXX $FLAGS -DTINY -DFPGA_EMULATOR -I $ONE $ONE/oneapi-target-4-run.cpp $LINK -o $ROOT/tests/_bin/oneapi_gemm_tiny
  # the oneAPI conv and capsule drivers: N-D operand layouts, constants read from the extents
  # (the copies under correctness/oneapi-integration: their relative include of Roofline.h resolves)
  ONEC="$REF/t2s/tests/correctness/oneapi-integration"
  $CXX $FLAGS -DTINY -DFPGA_EMULATOR -I $ONEC $ONEC/oneapi-target-5-run.cpp $LINK -o $ROOT/tests/_bin/oneapi_conv_tiny
  $CXX $FLAGS -DTINY -DFPGA_EMULATOR -I $ONEC $ONEC/oneapi-target-6-run.cpp $LINK -o $ROOT/tests/_bin/oneapi_capsule_tiny
  # the PEPPERS BLAS driver (sgemm with alpha/beta), A10 release constants with its own 4x4x4 outer loops
  BLAS="$REF/t2s/peppers/blas/level3/gemm/release/a10"
  $CXX $FLAGS -I $BLAS $BLAS/sgemm-run-fpga.cpp $STUBS/blas-gemm.cpp $LINK -o $ROOT/tests/_bin/blas_sgemm_a10
  # the PEPPERS SYRK driver over the folded-output syrk interface (S10 release constants: n = 768, k = 1024)
  SYRK="$REF/t2s/peppers/blas/level3/syrk/release/s10"
  $CXX $FLAGS -iquote $ROOT/include -I $SYRK $SYRK/ssyrk-run-fpga.cpp $STUBS/blas-syrk.cpp $STUBS/syrk-interface.cpp $LINK -o $ROOT/tests/_bin/blas_ssyrk_s10
  # the SYRK design's own driver: checks the folded 6-D output element by element (C not symmetric here)
  $CXX $FLAGS -DTINY -I $PERF/syrk $PERF/syrk/syrk-run-fpga.cpp $STUBS/syrk-interface.cpp $LINK -o $ROOT/tests/_bin/syrk_tiny
  # the GER design's driver (tiled 6-D output checked element by element)
  $CXX $FLAGS -DTINY -I $PERF/ger $PERF/ger/ger-run-fpga.cpp $STUBS/ger-interface.cpp $LINK -o $ROOT/tests/_bin/ger_tiny
  # the GPU-flow drivers, written against the Level Zero helper layer (util/l0_rt_helpers.h): this
  # repository's header of the same name and API stands in for it; -DITER=1 is the reference's
  # correctness mode (tests.sh:40), sizes are the GPU design's (2048^3 GEMM, 4 x 256 x 64 x 64 conv, ...)
  L0="-O3 -I $ROOT/include/l0 -DITER=1"
  $CXX $FLAGS $L0 -I $PERF/gemm    $PERF/gemm/gemm-run-gpu.cpp       $STUBS/l0_shim.cpp $LINK -o $ROOT/tests/_bin/gemm_gpu_flow
  $CXX $FLAGS $L0 -I $PERF/conv    $PERF/conv/conv-run-gpu.cpp       $STUBS/l0_shim.cpp $LINK -o $ROOT/tests/_bin/conv_gpu_flow
  $CXX $FLAGS $L0 -I $PERF/capsule $PERF/capsule/capsule-run-gpu.cpp $STUBS/l0_shim.cpp $LINK -o $ROOT/tests/_bin/capsule_gpu_flow
  # the CM-flow drivers (CmDevice / CmSurface2D / CmQueue ...): include/cm stands in for the CM runtime headers
  CM="-O3 -I $ROOT/include/cm -DITER=1"
  $CXX $FLAGS $CM -I $PERF/gemm    $PERF/gemm/gemm-run-gpu-cm.cpp       $STUBS/l0_shim.cpp $LINK -o $ROOT/tests/_bin/gemm_cm_flow
  $CXX $FLAGS $CM -I $PERF/conv    $PERF/conv/conv-run-gpu-cm.cpp       $STUBS/l0_shim.cpp $LINK -o $ROOT/tests/_bin/conv_cm_flow
  $CXX $FLAGS $CM -I $PERF/capsule $PERF/capsule/capsule-run-gpu-cm.cpp $STUBS/l0_shim.cpp $LINK -o $ROOT/tests/_bin/capsule_cm_flow
  # performance mode of the same drivers (no -DTINY: the A10 design constants and problem sizes),
  # with this repository's implementation of the Roofline.h helpers in place of Roofline.cpp
  SHIM="$ROOT/t2sp_b200/csrc/roofline_shim.cpp"
  $CXX $FLAGS -I $PERF/gemm    $PERF/gemm/gemm-run-fpga.cpp       $STUBS/gemm-interface.cpp    $SHIM $LINK -o $ROOT/tests/_bin/gemm_large_a10
  $CXX $FLAGS -I $PERF/conv    $PERF/conv/conv-run-fpga.cpp       $STUBS/conv-interface.cpp    $SHIM $LINK -o $ROOT/tests/_bin/conv_large_a10
  $CXX $FLAGS -I $PERF/capsule $PERF/capsule/capsule-run-fpga.cpp $STUBS/capsule-interface.cpp $SHIM $LINK -o $ROOT/tests/_bin/capsule_large_a10
  # a caller written with the reference tree's Halide::Runtime::Buffer class: the device interface table in use
  $CXX $FLAGS -O1 $ROOT/tests/drivers/runtime_buffer_flow.cpp $LINK -o $ROOT/tests/_bin/runtime_buffer_flow
fi
echo "reference drivers built"
