// NOT COMPILED: no JDK, Kotlin compiler or Gradle exists in the image this repository was built in.
// Written against ir/src/commonMain/kotlin/io/tlaloc/ir/recognizer/kernel/{KernelTemplate, KernelDescriptor,
// KernelTarget}.kt and ir/.../PagedAttentionAttrs.kt of the reference.
package io.tlaloc.ir.recognizer.kernel

import io.tlaloc.core.BF16
import io.tlaloc.core.ExperimentalTlalocApi
import io.tlaloc.core.F32
import io.tlaloc.core.F8E4M3FN
import io.tlaloc.ir.OpKind
import io.tlaloc.ir.PagedAttentionAttrs

/** Positions per context slice the emitter sizes the scratch result for (StablehloEmitter.kt:104). */
private const val SLICE = 256

/**
 * The paged-attention selector for [KernelTarget.NVIDIA_B200]: claims `PAGED_ATTENTION` and lowers it to the
 * typed-FFI custom call `@tlaloc_paged_attention` that libtlaloc_kernels.so (the B200 build) registers, with the
 * reference handler's wire format (triton/kernels/paged_attention.cu:5-17): operands query, keyCache, valueCache,
 * blockTables, seqLens (+ keep); results out and one XLA-owned scratch `[S, R, H, D + 2]`, `S = ceil(M * bs / 256)`.
 *
 * What it claims beyond [PagedAttentionKernel] (the GB10 / KPTX template): bf16 as well as f32 queries and outputs;
 * f32, bf16 and f8e4m3fn pools; rows that share a block table; a `sliding_window`; a `keep` operand.  The B200
 * kernels use at most `S` slices and mark nothing they do not use, so an unchanged emitter's scratch sizing holds.
 *
 * Declines anything [PagedAttentionAttrs] refuses, a head dimension above 256 (the kernels' limit), and any target
 * other than B200.  Like every claiming template of a first-class op, declining leaves the op's own gather-composed
 * emission in place.
 */
@ExperimentalTlalocApi
val B200PagedAttentionKernel: KernelTemplate = KernelTemplate { node, target ->
    if (target != KernelTarget.NVIDIA_B200) return@KernelTemplate null
    if (node.op != OpKind.PAGED_ATTENTION) return@KernelTemplate null
    val parsed = runCatching { PagedAttentionAttrs.parse(node, "B200PagedAttentionKernel") }
        .getOrNull() ?: return@KernelTemplate null
    val q = node.operands[0].type.dtype
    val kv = node.operands[1].type.dtype
    if (q != F32 && q != BF16) return@KernelTemplate null
    if (node.type.dtype != q) return@KernelTemplate null
    if (kv != F32 && kv != BF16 && kv != F8E4M3FN) return@KernelTemplate null
    if (node.operands[2].type.dtype != kv) return@KernelTemplate null
    if (parsed.headDim > 256) return@KernelTemplate null
    val context = parsed.maxBlocksPerSeq * parsed.blockSize
    val slices = (context + SLICE - 1) / SLICE
    KernelDescriptor(
        kernelName = "tlaloc_paged_attention",
        vendor = "tlaloc",
        targetArch = "b200",
        customCallAttrs = buildMap {
            put("scale", parsed.scale)
            parsed.slidingWindow?.let { put(PagedAttentionAttrs.SLIDING_WINDOW, it) }
        },
        typedFfi = true,
        scratchResults = listOf(listOf(slices, parsed.numSeqs, parsed.numHeads, parsed.headDim + 2)),
    )
}
