/*
 * fa2_b200 — hooks for tests and measurements. Not part of the attention path: nothing a host
 * runtime binds for the forward or backward call is declared here (that is fa2_b200.h). Neither hook
 * has a counterpart in erfanzar/jax-flash-attn2, whose Triton launches expose no status or per-kernel
 * timing (jax_flash_attn2/flash_attention_triton/_backward_triton.py:1049-1154).
 */
#ifndef FA2_B200_DEBUG_H_
#define FA2_B200_DEBUG_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Reads and clears the device status word written by a kernel whose bounded wait ran out
 * (0 = no time-out seen). Synchronises the stream; meant for tests and debugging. */
int fa2_debug_device_status(void* cuda_stream);

/* Profiling hook: arms four CUDA events (cudaEvent_t cast to void*) for the next fa2_bwd call on
 * this thread. They are recorded on that call's stream before the rowsum pre-pass, before the
 * main kernel, after it and after the dq conversion, so a caller can time each kernel of the
 * backward (the three launches that replace _backward_triton.py:1049-1154). NULL disarms. */
int fa2_debug_bwd_stage_events(void* const* events);

#ifdef __cplusplus
}
#endif
#endif /* FA2_B200_DEBUG_H_ */
