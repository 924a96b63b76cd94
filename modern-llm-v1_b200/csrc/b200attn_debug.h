/*
 * Tuning builds only (-DB200ATTN_PROBE): the kernels then record clock64() at numbered points of the first CTA
 * (B200ATTN_STAMP in ptx.cuh) and, per CTA, the SM id and the begin / end times (B200ATTN_TRACE_*).  These three
 * calls copy those arrays to the host after a launch.  They are not part of the library's interface: the regular
 * build neither records anything nor exports these symbols, and include/b200attn.h does not declare them.
 */
#ifndef B200ATTN_DEBUG_H_
#define B200ATTN_DEBUG_H_
#ifdef B200ATTN_PROBE
#ifdef __cplusplus
extern "C" {
#endif
/* the first n (<= 512) phase stamps of the last launch, in SM clocks */
int b200attn_debug_read_probe(long long* host, int n);
/* per CTA of the last launches: SM id, begin and end (globaltimer, ns); kernel k's CTAs start at 2048 * k */
int b200attn_debug_read_trace(unsigned long long* host, int n_ctas);
/* the same two points in SM clocks */
int b200attn_debug_read_trace_clk(long long* host, int n_ctas);
#ifdef __cplusplus
}
#endif
#endif
#endif
