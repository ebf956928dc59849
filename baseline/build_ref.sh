#!/usr/bin/env bash
# Builds the reference's CUDA programs, unmodified, for sm_100 into baseline/_ref/bin (git-ignored).
# They are the same-box baselines for the micro-benchmarks: contiguous cudaMemcpyPeerAsync transfers,
# the HBM stressor, the decode KV-scan stressors, memhog and the PCIe memcpy worker.
# cpu_client.cc / gpu_server.cu need <infiniband/verbs.h> and are skipped when it is missing.
set -u
REF="${1:-${SKYGDR_REFERENCE_DIR:-}}"
if [ -z "$REF" ] || [ ! -d "$REF" ]; then echo "usage: build_ref.sh <path to the reference checkout> (or set SKYGDR_REFERENCE_DIR)" >&2; exit 2; fi
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref/bin"
mkdir -p "$OUT"
ARCH="-gencode arch=compute_100,code=sm_100"
ok=0; fail=0
for f in llm_problem_analysis/kv_nvlink_transfer.cu llm_problem_analysis/kv_nvlink_transfer_trace.cu \
         llm_problem_analysis/decode_hbm_stress.cu llm_problem_analysis/decode_transformer_kvcache_stress.cu \
         llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu src/gpu_be_memhog_task.cu src/gpu_be_pcie_memcpy_task.cu; do
  name="$(basename "$f" .cu)"
  if nvcc -O3 -std=c++17 $ARCH "$REF/$f" -o "$OUT/$name" 2> "$OUT/$name.build.log"; then ok=$((ok+1)); else fail=$((fail+1)); echo "build failed: $f (see $OUT/$name.build.log)"; fi
done
if [ -f /usr/include/infiniband/verbs.h ]; then
  g++ -O2 -std=c++14 "$REF/src/cpu_client.cc" -o "$OUT/cpu_client" -libverbs -lpthread 2> "$OUT/cpu_client.build.log" || echo "cpu_client: build failed"
else
  echo "cpu_client / gpu_server: skipped (no infiniband/verbs.h on this image)"
fi
echo "reference programs built: $ok ok, $fail failed -> $OUT"
