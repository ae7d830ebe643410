// Test infrastructure, not product code: exports the typed-FFI handler of the REFERENCE's own CUDA paged-attention
// kernel (triton/kernels/paged_attention.cu:1334-1446, PagedAttentionHandler, which sits in an unnamed namespace of
// that file) so that tests and the benchmark can run the reference's kernel, built for sm_100a from its own sources
// where they lie, on the same GPU as this library's.  The reference source is included at build time by
// oracle/build_ref.sh (-I <reference>/triton/kernels); nothing of it is copied into this repository.
#include "paged_attention.cu"

extern "C" __attribute__((visibility("default"))) void* tlaloc_ref_paged_attention_handler(void)
{
  return reinterpret_cast<void*>(&PagedAttentionHandler);
}
