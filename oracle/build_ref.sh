#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY (never part of the product path).
#
# Builds the unmodified reference MoE layer (kernel/*.cu, kernel/*.cpp of the
# reference checkout) into oracle/_ref/libref_moe.so, compiling the sources
# where they lie.  No reference source is copied into this repository; only
# object files and the shared library are written, all under oracle/_ref/.
#
# usage: oracle/build_ref.sh [REFERENCE_DIR]      (default /root/reference)
#
# The library exports the reference's own entry point `__tvm_ffi_run`
# (kernel/moe_fp8.cu:3674) and is loaded with tvm_ffi.load_module().
set -euo pipefail
REF="${1:-/root/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT/inc/flashinfer/trtllm/batched_gemm"
SP="$(python -c 'import sysconfig; print(sysconfig.get_paths()["purelib"])')"
FI="$SP/flashinfer"
TVM="$SP/tvm_ffi"
BMM="$(ls -d "$SP"/flashinfer_cubin/cubins/*/batched_gemm-* | head -n1)"
# The reference includes the generated BMM headers below flashinfer/trtllm/batched_gemm/.
ln -sfn "$BMM/include/trtllmGen_bmm_export" "$OUT/inc/flashinfer/trtllm/batched_gemm/trtllmGen_bmm_export"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
ARCH="-gencode arch=compute_100a,code=sm_100a"
COMMON="-std=c++17 -O2 $ARCH --expt-relaxed-constexpr -Xcompiler -fPIC -w"
TLLM_DEFS="-DTLLM_ENABLE_CUDA -DTLLM_GEN_EXPORT_INTERFACE -DTLLM_GEN_EXPORT_FLASHINFER -DTLLM_GEN_GEMM_CUBIN_PATH=\"$BMM\""
TLLM_INC="-I $OUT/inc -I $FI/data/include -I $FI/data/csrc/nv_internal -I $FI/data/csrc/nv_internal/include -I $BMM/include -I $FI/data/spdlog/include"
K="$REF/kernel"
pids=()
# The two slow objects are rebuilt only when their reference source is newer.
if [ ! -f "$OUT/cutlass_gemm.o" ] || [ "$K/cutlass_gemm.cu" -nt "$OUT/cutlass_gemm.o" ]; then
( $NVCC $COMMON -I "$FI/data/cutlass/include" -I "$FI/data/cutlass/tools/util/include" \
    -c "$K/cutlass_gemm.cu" -o "$OUT/cutlass_gemm.o" ) & pids+=($!)
fi
if [ ! -f "$OUT/trtllm_runner.o" ] || [ "$K/trtllm_batched_gemm_runner.cu" -nt "$OUT/trtllm_runner.o" ]; then
( $NVCC $COMMON $TLLM_DEFS $TLLM_INC -c "$K/trtllm_batched_gemm_runner.cu" -o "$OUT/trtllm_runner.o" ) & pids+=($!)
fi
# moe_fp8.cu is compiled through ref_harness.cu, which includes it unchanged and appends
# test entry points for the reference's routing / dispatch kernels.
# MOE_TRTLLM_BMM_CONFIG is one of the reference's own #ifndef knobs (kernel/moe_fp8.cu:87-89).  Its
# default, 364, is a position in the kernel table generated for flashinfer 0.6.8.post1; in this
# image's flashinfer_cubin table position 364 is an e4m3-output, 8-token-tile kernel, and running
# it with the reference's bf16 / 64-token-tile arguments made an illegal memory access.  -1 makes
# the adapter ask the runner for its default valid configuration (kernel/trtllm_fp8_bmm.cu:88-98).
REF_KNOBS="${REF_KNOBS:--DMOE_TRTLLM_BMM_CONFIG=-1}"
( $NVCC $COMMON $REF_KNOBS -I "$K" -I "$TVM/include" -I "$TVM/3rdparty/dlpack/include" -c "$HERE/ref_harness.cu" -o "$OUT/moe_fp8.o" ) & pids+=($!)
( $NVCC $COMMON $TLLM_DEFS $TLLM_INC -c "$K/trtllm_fp8_bmm.cu" -o "$OUT/trtllm_fp8_bmm.o" ) & pids+=($!)
for f in envUtils logger stringUtils tllmException; do
  ( g++ -std=c++17 -O2 -fPIC -w $TLLM_DEFS $TLLM_INC -I /usr/local/cuda/include \
      -c "$K/$f.cpp" -o "$OUT/$f.o" ) & pids+=($!)
done
rc=0
for p in "${pids[@]}"; do wait "$p" || rc=1; done
[ $rc -eq 0 ] || { echo "reference build: a compile step failed" >&2; exit 1; }
g++ -shared -o "$OUT/libref_moe.so" "$OUT"/*.o \
    -L /usr/local/cuda/lib64 -lcudart -L "$TVM/lib" -ltvm_ffi \
    -Wl,-rpath,"$TVM/lib" -Wl,-rpath,/usr/local/cuda/lib64 \
    -L /usr/local/cuda/lib64/stubs -lcuda -ldl
echo "built $OUT/libref_moe.so"
