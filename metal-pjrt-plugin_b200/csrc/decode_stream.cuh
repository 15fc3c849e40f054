// The whole decode step as ONE persistent kernel (decode_stream.cu), as seen by decoder.cu.
#pragma once
#include <vector>

#include "tp.cuh"

namespace b200 {

struct DecodeStream;   // owns the repacked int4 weight stream, the stage table and the activations

// Builds the single-kernel path for this decoder when its shapes allow it (all projection
// widths multiples of 16, 16-byte-aligned buffers, a supported head_dim / group size, cache
// rows that allow 16-byte loads).  *out stays null, with B200_OK, when they do not: the
// caller then keeps the kernel-per-operator path.  `vocab_full` is the embedding table's row
// count.  The int4 projections are copied once into the kernel's own streaming layout
// (one contiguous record per 16 rows x 512 inputs, in the order each CTA consumes them).
b200_status DecodeStreamCreate(b200_context* ctx, const b200_decoder_config& cfg,
                               const std::vector<b200_decoder_layer>& layers, const void* embed,
                               const void* final_norm, const void* lm_head, int64_t vocab_full, b200_tp* tp,
                               DecodeStream** out);
void DecodeStreamDestroy(DecodeStream* ds);
// Batches the single kernel takes (the inputs of every row must fit one CTA's shared memory).
bool DecodeStreamSupports(const DecodeStream* ds, int batch);
// One step: tokens int32 [batch], pos int32 [1], logits f32 [batch, vocab] (device).  With
// next_token != null the kernel also writes argmax(logits) per row (int32 [batch]).
b200_status DecodeStreamStep(DecodeStream* ds, cudaStream_t stream, const int32_t* tokens, const int32_t* pos,
                             float* logits, int32_t* next_token, int batch);
// Bytes of device memory the repacked weights take.
size_t DecodeStreamPackedBytes(const DecodeStream* ds);
// Per-stage tracing (see b200_decoder_trace in the C header).
b200_status DecodeStreamTrace(DecodeStream* ds, bool enable);
b200_status DecodeStreamTraceRead(DecodeStream* ds, unsigned long long* out, int64_t capacity, int* ctas, int* stages,
                                  int* stage_types);

}  // namespace b200
