// Device entry points of the op implementations. Each group lives in its own
// translation unit (relocatable device code) so the compiler works on them
// separately and in parallel.
#pragma once
#include "dev_common.cuh"

namespace arkb {
struct GemmPipe;
__device__ void run_ewise(const EwiseArgs &a, int p, int P, unsigned long long iter_no);
__device__ void run_reduce(const ReduceArgs &a, int p, int P, char *smem);
__device__ void run_rowop(const RowOpArgs &a, int p, int P, char *smem, CtaCtl *ctl, DeviceState *st, int stage_idx,
                          unsigned long long wait_limit);
__device__ void run_transpose(const TransposeArgs &a, int p, int P, char *smem);
__device__ void run_embed(const EmbedArgs &a, int p, int P);
// `g` may be a copy of the stage record in shared memory; `gmaps` is the record in global memory (tensor maps are read there)
__device__ void run_gemm(const GemmArgs &g, const GemmArgs *gmaps, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl,
                         DeviceState *st, int stage_idx, unsigned long long spin_limit);
__device__ void run_gemm_pair(const GemmArgs &g, const GemmArgs *gmaps, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl,
                              DeviceState *st, int stage_idx, unsigned long long spin_limit);
__device__ void run_splitk_reduce(const SplitKReduceArgs &a, int p, int P);
__device__ void run_gemv(const GemvArgs &a, int p, int P, char *smem, const LaunchParams &LP, unsigned long long iter_no);
__device__ void run_decode_attn(const DecodeAttnArgs &a, int p, int P, char *smem);
__device__ void run_prefill_attn(const PrefillAttnArgs &a, const PrefillAttnArgs *amaps, int p, int P, char *smem, CtaCtl *ctl,
                                 DeviceState *st, int stage_idx, unsigned long long spin_limit);
__device__ void run_gemm_simt(const GemmSimtArgs &g, int p, int P, char *smem);
__device__ void run_put(const PutArgs &a, int p, int P, unsigned long long iter_no);
__device__ void run_packet(const LaunchParams &P, const PacketArgs &a, int p, int Pn, unsigned long long iter_no, CtaCtl *ctl, int stage);
__device__ void run_packet_reduce(const LaunchParams &P, const PacketReduceArgs &a, int p, int Pn, unsigned long long iter_no, CtaCtl *ctl,
                                  int stage);
__device__ void run_allreduce(const LaunchParams &P, const AllReduceArgs &a, int p, int Pn, unsigned long long iter_no);
}  // namespace arkb
