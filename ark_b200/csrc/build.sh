#!/bin/bash
# Builds libark_b200.so: the sm_100a loop kernel (relocatable device code, one
# translation unit per op group, compiled in parallel) plus the host runtime.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="${ARKB_OUT:-$HERE/../lib}"
mkdir -p "$OUT/obj"
NVCC=${NVCC:-nvcc}
ARCH="-gencode arch=compute_100a,code=sm_100a"
CUFLAGS="$ARCH ${ARKB_DEFS:-} -lineinfo -O3 -std=c++17 -rdc=true -maxrregcount=128 -Xcompiler -fPIC ${ARKB_PTXAS_V:+-Xptxas -v}"
pids=()
for f in loop_kernel dev_ewise dev_reduce dev_gemm dev_gemv dev_attn dev_attn_prefill dev_comm; do
  if [ "$HERE/$f.cu" -nt "$OUT/obj/$f.o" ] || [ -n "$(find "$HERE" -maxdepth 1 \( -name '*.h' -o -name '*.cuh' \) -newer "$OUT/obj/$f.o" 2>/dev/null)" ] || [ ! -f "$OUT/obj/$f.o" ]; then
    $NVCC $CUFLAGS -dc "$HERE/$f.cu" -o "$OUT/obj/$f.o" > "$OUT/obj/$f.log" 2>&1 &
    pids+=($!)
  fi
done
# stand-alone CUDA translation units (no relocatable device code)
for f in noalloc_gemv; do
  $NVCC $ARCH ${ARKB_DEFS:-} -lineinfo -O3 -std=c++17 -Xcompiler -fPIC -I"$HERE/../../include" -c "$HERE/$f.cu" -o "$OUT/obj/$f.o" > "$OUT/obj/$f.log" 2>&1 &
  pids+=($!)
done
HOSTSRC=""
for f in "$HERE"/*.cpp; do [ -f "$f" ] && HOSTSRC="$HOSTSRC $f"; done
for f in $HOSTSRC; do
  b=$(basename "$f" .cpp)
  g++ -O2 -std=c++17 -fPIC -I/usr/local/cuda/include -I"$HERE/../../include" -c "$f" -o "$OUT/obj/$b.o" > "$OUT/obj/$b.log" 2>&1 &
  pids+=($!)
done
fail=0
for p in "${pids[@]}"; do wait $p || fail=1; done
cat "$OUT"/obj/*.log
[ $fail -eq 0 ] || { echo "compile failed"; exit 1; }
$NVCC $ARCH -dlink -Xcompiler -fPIC "$OUT"/obj/loop_kernel.o "$OUT"/obj/dev_*.o -o "$OUT/obj/dlink.o"
g++ -shared -fPIC -o "$OUT/libark_b200.so" "$OUT"/obj/*.o -L/usr/local/cuda/lib64 -lcudart_static -ldl -lrt -lpthread
echo "built $OUT/libark_b200.so"
