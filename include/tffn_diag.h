/* tffn_diag.h — profiling and tuning aids of libtffn.so. None of these has a counterpart in the
 * reference and none is needed to run inference; they exist to measure where a decode step's time
 * goes (per-kernel events, in-kernel timestamps, ablation). Kept apart from tffn.h so that a binding
 * of the inference path does not have to carry them.
 */
#ifndef TFFN_DIAG_H
#define TFFN_DIAG_H
#include "tffn.h"
#ifdef __cplusplus
extern "C" {
#endif

/* Timing aid: kernel classes (bit i = class i of tffn_profile_class_name) that the batched path
 * skips from now on. The step then computes garbage; the drop in step time is what that class costs
 * inside the overlapped (dependent-launch, graph) schedule, which per-kernel events cannot show.
 * 0 restores normal operation. */
int tffn_session_set_ablation(tffn_session* s, unsigned mask);
/* Per-kernel timing for benchmarks: while enabled, every kernel launch of the session is
 * bracketed by CUDA events on the session's stream (this serialises kernels that would
 * otherwise overlap, so never time throughput with it on). tffn_session_profile_read returns the
 * number of kernel classes and fills ms[i] (device time) and launches[i] for i < cap;
 * tffn_profile_class_name(i) names class i. No counterpart in the reference. */
int tffn_session_profile(tffn_session* s, int enable);
int tffn_session_profile_read(tffn_session* s, float* ms, int32_t* launches, int cap);
const char* tffn_profile_class_name(int cls);
/* Profiling aid (no counterpart in the reference): runs three batched decode steps of slots
 * 0..n_seqs-1 in the session's launch mode (the sequences advance by three tokens) and reports the
 * timeline of the last one. out[i*7] = kernel class of launch i (tffn_profile_class_name), then the
 * minimum and maximum over the launch's CTAs of: kernel entry, return from the grid-dependency wait,
 * exit (globaltimer, ns). Unlike per-kernel events this shows the overlapped schedule as it runs.
 * If trace_out is not NULL and launch number trace_launch is a tensor-core GEMM of at most trace_ctas
 * CTAs, trace_out[cta*64 + k] receives that launch's per-CTA phase timestamps (k as documented for
 * tffn_op_gemm_trace). Returns the number of launches (at most max_launches are recorded). */
int tffn_session_timeline(tffn_session* s, int n_seqs, uint64_t* out, int max_launches, int trace_launch,
                          uint64_t* trace_out, int trace_ctas);
/* tffn_op_gemm, and additionally returns 64 device timestamps (globaltimer, ns) per CTA in trace[trace_ctas*64]
 * (CTA order: split-major, then token tile, then row tile): 0 start, 1 weight boxes requested,
 * 2 dependency wait over, 3 last MMA issued, 4 accumulator complete, 5 epilogue done, 6 cluster
 * barrier passed, 7 cluster reduction done, 8 end, 16+i pipeline stage i arrived. A profiling aid with
 * no counterpart in the reference. */
int tffn_op_gemm_trace(int device, const uint16_t* X, const uint16_t* W, float* out, int T, int N, int K, int splits,
                       uint64_t* trace, int trace_ctas);
/* tffn_op_swiglu_bs1, and additionally returns 16 device timestamps (globaltimer, ns) per CTA of a second, warm
 * launch in trace[trace_ctas*16] (trace_ctas >= SM count): 0 start, 1 RMSNorm done, 2 first record
 * arrived, 3 last record consumed, 4 CTA partial written, 5 group ticket taken, 6 group fold done,
 * 7 residual updated. A profiling aid with no counterpart in the reference. */
int tffn_op_swiglu_bs1_trace(int device, const uint16_t* h_in, const uint16_t* norm_w, const uint16_t* packed_base,
                             const uint16_t* packed_expert, float expert_scale, float eps, int H, int I, uint16_t* h_out,
                             uint64_t* trace, int trace_ctas);

#ifdef __cplusplus
}
#endif
#endif
