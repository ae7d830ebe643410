// NOT COMPILED: no JDK, Kotlin compiler or Gradle exists in the image this repository was built in.
// Written against include/tlaloc_b200.h (ABI version 1) and the reference's FFM conventions
// (runtime-cuda/src/jvmMain/kotlin/io/tlaloc/runtime/cuda/CudaDriverFfm.kt:62-103).
package io.tlaloc.runtime.cuda

import java.lang.foreign.Arena
import java.lang.foreign.FunctionDescriptor
import java.lang.foreign.Linker
import java.lang.foreign.MemorySegment
import java.lang.foreign.SymbolLookup
import java.lang.foreign.ValueLayout.ADDRESS
import java.lang.foreign.ValueLayout.JAVA_FLOAT
import java.lang.foreign.ValueLayout.JAVA_INT
import java.lang.foreign.ValueLayout.JAVA_LONG
import java.lang.invoke.MethodHandle
import java.nio.file.Path

/** A status other than TLALOC_B200_OK, with the library's message for the calling thread. */
class TlalocB200Exception(val status: Int, message: String) : RuntimeException(message)

/**
 * libtlaloc_kernels.so's flat C functions as method handles.  Device pointers travel as `Long` (what
 * [CudaDriverFfm.memAlloc] returns), the stream as the CUstream address, sizes as `Int`/`Long`; every call only
 * enqueues work on the stream.  One instance per process is enough; it is thread-safe (the library keeps its error
 * message per thread).
 */
class TlalocB200Ffm private constructor(arena: Arena, library: Path) {
    companion object {
        private val LINKER: Linker = Linker.nativeLinker()
        const val OK = 0
        const val INVALID_ARGUMENT = -1
        const val UNSUPPORTED = -2
        const val INTERNAL = -3

        // Element types, numbered as XLA_FFI_DataType.
        const val S8 = 2
        const val S32 = 4
        const val F32 = 11
        const val BF16 = 16
        const val F8E4M3FN = 20

        const val GEMM_EXACT = 1
        const val GEMM_X_F32_EXACT = 2
        const val GEMM_WEIGHTS_CONST = 4
        const val GEMM_I8_MMA = 8
        const val GEMM_X_PLANES = 16

        fun load(arena: Arena, library: Path): TlalocB200Ffm {
            val lib = TlalocB200Ffm(arena, library)
            val v = lib.abiVersion.invokeExact() as Int
            require(v == 1) { "$library has ABI version $v, these bindings were written for 1" }
            return lib
        }
    }

    private val lookup: SymbolLookup = SymbolLookup.libraryLookup(library, arena)

    private fun handle(symbol: String, descriptor: FunctionDescriptor): MethodHandle =
        LINKER.downcallHandle(
            lookup.find(symbol).orElseThrow { IllegalStateException("$library does not export $symbol") },
            descriptor,
        )

    private fun ptr(address: Long): MemorySegment = MemorySegment.ofAddress(address)

    private val abiVersion = handle("tlaloc_b200_abi_version", FunctionDescriptor.of(JAVA_INT))
    private val lastError = handle("tlaloc_b200_last_error", FunctionDescriptor.of(ADDRESS))
    private val init = handle("tlaloc_b200_init", FunctionDescriptor.of(JAVA_INT))
    private val deviceStatus = handle("tlaloc_b200_device_status", FunctionDescriptor.of(JAVA_INT))
    private val setOrderFaithful = handle("tlaloc_b200_set_order_faithful", FunctionDescriptor.of(JAVA_INT, JAVA_INT))
    private val launchCount = handle("tlaloc_b200_launch_count", FunctionDescriptor.of(JAVA_LONG))
    private val paSplits = handle(
        "tlaloc_b200_paged_attention_splits",
        FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT),
    )
    private val paScratchBytes = handle(
        "tlaloc_b200_paged_attention_scratch_bytes",
        FunctionDescriptor.of(JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT),
    )
    private val pagedAttention = handle(
        "tlaloc_b200_paged_attention",
        FunctionDescriptor.of(
            JAVA_INT,
            ADDRESS, JAVA_INT,                    // query, q_dtype
            ADDRESS, ADDRESS, JAVA_INT,           // key_cache, value_cache, kv_dtype
            ADDRESS, ADDRESS,                     // block_tables, seq_lens
            ADDRESS, JAVA_INT,                    // keep, keep_chunks
            ADDRESS, JAVA_INT,                    // out, out_dtype
            ADDRESS,                              // lse
            ADDRESS, JAVA_INT,                    // scratch, splits
            JAVA_INT, JAVA_INT, JAVA_INT,         // num_rows, num_heads, head_dim
            JAVA_INT, JAVA_INT, JAVA_INT,         // num_blocks, block_size, num_kv_heads
            JAVA_INT, JAVA_INT,                   // max_blocks_per_seq, num_tables
            JAVA_FLOAT, JAVA_INT,                 // scale, sliding_window
            ADDRESS,                              // stream
        ),
    )
    private val paStaticBytes = handle("tlaloc_b200_paged_attention_static_scratch_bytes", FunctionDescriptor.of(JAVA_LONG))
    private val pagedAttentionStatic = handle(
        "tlaloc_b200_paged_attention_static",
        FunctionDescriptor.of(
            JAVA_INT,
            ADDRESS, JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS,
            JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_FLOAT, JAVA_INT, ADDRESS,
        ),
    )
    private val kvCacheWrite = handle(
        "tlaloc_b200_kv_cache_write",
        FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS),
    )
    private val gemmScratchBytes = handle(
        "tlaloc_b200_int8_gemm_scratch_bytes", FunctionDescriptor.of(JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT),
    )
    private val int8Gemm = handle(
        "tlaloc_b200_int8_gemm",
        FunctionDescriptor.of(
            JAVA_INT,
            ADDRESS, JAVA_INT,                    // x, x_dtype
            ADDRESS, ADDRESS, ADDRESS,            // codes, scales, residual
            ADDRESS, JAVA_INT,                    // y, y_dtype
            ADDRESS, JAVA_LONG,                   // scratch, scratch_bytes
            JAVA_INT, JAVA_INT, JAVA_INT,         // m, k, n
            JAVA_INT, ADDRESS,                    // flags, stream
        ),
    )
    private val int8GemmSwiglu = handle(
        "tlaloc_b200_int8_gemm_swiglu",
        FunctionDescriptor.of(
            JAVA_INT,
            ADDRESS, JAVA_INT,                    // x, x_dtype
            ADDRESS, ADDRESS,                     // codes (gate|up interleaved in blocks of 128 + 128), scales
            ADDRESS, JAVA_INT,                    // y [M, N / 2], y_dtype
            ADDRESS, JAVA_LONG,                   // scratch, scratch_bytes
            JAVA_INT, JAVA_INT, JAVA_INT,         // m, k, n
            JAVA_INT, ADDRESS,                    // flags, stream
        ),
    )
    private val denseGemmExact = handle(
        "tlaloc_b200_dense_gemm_exact",
        FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS),
    )
    private val embedding = handle(
        "tlaloc_b200_embedding",
        FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS),
    )
    private val rmsnorm = handle(
        "tlaloc_b200_rmsnorm",
        FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_FLOAT, ADDRESS),
    )
    private val ropeKvWrite = handle(
        "tlaloc_b200_rope_kv_write",
        FunctionDescriptor.of(
            JAVA_INT,
            ADDRESS, ADDRESS, ADDRESS,            // q, k, v
            ADDRESS, ADDRESS, ADDRESS, ADDRESS,   // positions, cos, sin, slot_mapping
            ADDRESS, JAVA_INT,                    // q_out, q_out_dtype
            ADDRESS, ADDRESS, JAVA_INT,           // key_cache, value_cache, kv_dtype
            JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT,  // num_tokens, num_heads, num_kv_heads, head_dim
            JAVA_INT, JAVA_INT,                   // num_slots, max_pos
            JAVA_INT, JAVA_INT, JAVA_INT,         // ld_q, ld_k, ld_v
            ADDRESS,
        ),
    )
    private val swiglu = handle(
        "tlaloc_b200_swiglu",
        FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS),
    )
    private val argmax = handle(
        "tlaloc_b200_argmax", FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS),
    )
    private val peerAlloc = handle("tlaloc_b200_peer_alloc", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS))
    private val peerOpen = handle("tlaloc_b200_peer_open", FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS))
    private val peerClose = handle("tlaloc_b200_peer_close", FunctionDescriptor.of(JAVA_INT, ADDRESS))
    private val peerFree = handle("tlaloc_b200_peer_free", FunctionDescriptor.of(JAVA_INT, ADDRESS))
    private val peerAllReduce = handle(
        "tlaloc_b200_peer_allreduce_f32",
        FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_INT, JAVA_LONG, ADDRESS),
    )
    private val peerAllReduceNorm = handle(
        "tlaloc_b200_peer_allreduce_rmsnorm_f32",
        FunctionDescriptor.of(
            JAVA_INT, ADDRESS, JAVA_LONG, JAVA_LONG, JAVA_LONG, ADDRESS, ADDRESS, JAVA_FLOAT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS,
        ),
    )
    private val peerReduceNormRows = handle(
        "tlaloc_b200_peer_reduce_rmsnorm_rows_f32",
        FunctionDescriptor.of(
            JAVA_INT, ADDRESS, JAVA_LONG, JAVA_LONG, JAVA_LONG, ADDRESS,   // bases, data_offset, norm_offset, flag_offset, state
            ADDRESS, ADDRESS, JAVA_FLOAT,                                  // own_rows, gain, eps
            JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS,     // rank, world, rows, cols, planes (0 | 1), stream
        ),
    )
    private val peerSumRows = handle(
        "tlaloc_b200_peer_sum_rows_f32",
        FunctionDescriptor.of(
            JAVA_INT, ADDRESS, JAVA_LONG, JAVA_LONG, ADDRESS,   // bases, partial_offset, flag_offset, state
            ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_FLOAT,     // residual, out, norm_out, gain, eps
            JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT,             // rank, world, rows, cols
            ADDRESS, JAVA_LONG, ADDRESS,                        // planes (or null), planes_bytes, stream
        ),
    )
    private val rmsnormPlanes = handle(
        "tlaloc_b200_rmsnorm_planes",
        FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_FLOAT, ADDRESS),
    )
    private val registerKernels = handle("TlalocRegisterKernels", FunctionDescriptor.of(ADDRESS, ADDRESS))
    private val ffiHandler = handle("tlaloc_b200_ffi_handler", FunctionDescriptor.of(ADDRESS, ADDRESS))

    private fun check(status: Int) {
        if (status == OK) return
        val msg = (lastError.invokeExact() as MemorySegment).reinterpret(512).getString(0)
        throw TlalocB200Exception(status, msg)
    }

    /** Kernel set-up for the current device; once per device, before any graph capture. */
    fun init() = check(init.invokeExact() as Int)

    /** 1 if a bounded device-side wait gave up since the last call. Synchronises with the device. */
    fun deviceStatus(): Int = deviceStatus.invokeExact() as Int

    /** Parity mode (the interpreter's own evaluation order in every operator); returns the previous setting. */
    fun setOrderFaithful(on: Boolean): Boolean = (setOrderFaithful.invokeExact(if (on) 1 else 0) as Int) != 0

    fun launchCount(): Long = launchCount.invokeExact() as Long

    /** The slice count the reference's emitter sizes its scratch result for: ceil(maxBlocksPerSeq * blockSize / 256). */
    fun pagedAttentionSplits(numRows: Int, numKvHeads: Int, numTables: Int, maxBlocksPerSeq: Int, blockSize: Int): Int =
        paSplits.invokeExact(numRows, numKvHeads, numTables, maxBlocksPerSeq, blockSize) as Int

    fun pagedAttentionScratchBytes(numRows: Int, numHeads: Int, headDim: Int, splits: Int): Long =
        paScratchBytes.invokeExact(numRows, numHeads, headDim, splits) as Long

    /** PAGED_ATTENTION; argument meaning as `io.tlaloc.ir.PagedAttentionAttrs` and include/tlaloc_b200.h. */
    @Suppress("LongParameterList")
    fun pagedAttention(
        query: Long, qDtype: Int, keyCache: Long, valueCache: Long, kvDtype: Int, blockTables: Long, seqLens: Long,
        keep: Long, keepChunks: Int, out: Long, outDtype: Int, lse: Long, scratch: Long, splits: Int,
        numRows: Int, numHeads: Int, headDim: Int, numBlocks: Int, blockSize: Int, numKvHeads: Int,
        maxBlocksPerSeq: Int, numTables: Int, scale: Float, slidingWindow: Int, stream: Long,
    ) = check(
        pagedAttention.invokeExact(
            ptr(query), qDtype, ptr(keyCache), ptr(valueCache), kvDtype, ptr(blockTables), ptr(seqLens), ptr(keep), keepChunks,
            ptr(out), outDtype, ptr(lse), ptr(scratch), splits, numRows, numHeads, headDim, numBlocks, blockSize, numKvHeads,
            maxBlocksPerSeq, numTables, scale, slidingWindow, ptr(stream),
        ) as Int,
    )

    fun pagedAttentionStaticScratchBytes(): Long = paStaticBytes.invokeExact() as Long

    /** The same operator with the split records in the library's built-in 16 MiB array: for callers that cannot allocate. */
    @Suppress("LongParameterList")
    fun pagedAttentionStatic(
        query: Long, qDtype: Int, keyCache: Long, valueCache: Long, kvDtype: Int, blockTables: Long, seqLens: Long,
        keep: Long, keepChunks: Int, out: Long, outDtype: Int, lse: Long,
        numRows: Int, numHeads: Int, headDim: Int, numBlocks: Int, blockSize: Int, numKvHeads: Int,
        maxBlocksPerSeq: Int, numTables: Int, scale: Float, slidingWindow: Int, stream: Long,
    ) = check(
        pagedAttentionStatic.invokeExact(
            ptr(query), qDtype, ptr(keyCache), ptr(valueCache), kvDtype, ptr(blockTables), ptr(seqLens), ptr(keep), keepChunks,
            ptr(out), outDtype, ptr(lse), numRows, numHeads, headDim, numBlocks, blockSize, numKvHeads, maxBlocksPerSeq,
            numTables, scale, slidingWindow, ptr(stream),
        ) as Int,
    )

    /** KV_CACHE_WRITE in place; negative slots are padding. */
    fun kvCacheWrite(pool: Long, poolDtype: Int, newKv: Long, newDtype: Int, slotMapping: Long, numTokens: Int, rowElems: Int, numSlots: Int, stream: Long) =
        check(kvCacheWrite.invokeExact(ptr(pool), poolDtype, ptr(newKv), newDtype, ptr(slotMapping), numTokens, rowElems, numSlots, ptr(stream)) as Int)

    fun int8GemmScratchBytes(m: Int, k: Int, n: Int): Long = gemmScratchBytes.invokeExact(m, k, n) as Long

    /** y = (cast(x) @ cast(codes)) * scales (+ residual): HfDecoderGraph.proj over a WeightQuant.INT8 weight. */
    @Suppress("LongParameterList")
    fun int8Gemm(
        x: Long, xDtype: Int, codes: Long, scales: Long, residual: Long, y: Long, yDtype: Int, scratch: Long, scratchBytes: Long,
        m: Int, k: Int, n: Int, flags: Int, stream: Long,
    ) = check(
        int8Gemm.invokeExact(ptr(x), xDtype, ptr(codes), ptr(scales), ptr(residual), ptr(y), yDtype, ptr(scratch), scratchBytes, m, k, n, flags, ptr(stream)) as Int,
    )

    /** silu(x @ gate) * (x @ up) over one weight [K, 2F] with gate and up interleaved in column blocks of 128 + 128 (mlpOut). */
    @Suppress("LongParameterList")
    fun int8GemmSwiglu(
        x: Long, xDtype: Int, codes: Long, scales: Long, y: Long, yDtype: Int, scratch: Long, scratchBytes: Long,
        m: Int, k: Int, n: Int, flags: Int, stream: Long,
    ) = check(
        int8GemmSwiglu.invokeExact(ptr(x), xDtype, ptr(codes), ptr(scales), ptr(y), yDtype, ptr(scratch), scratchBytes, m, k, n, flags, ptr(stream)) as Int,
    )

    fun denseGemmExact(x: Long, xDtype: Int, w: Long, wDtype: Int, y: Long, m: Int, k: Int, n: Int, flags: Int, stream: Long) =
        check(denseGemmExact.invokeExact(ptr(x), xDtype, ptr(w), wDtype, ptr(y), m, k, n, flags, ptr(stream)) as Int)

    fun embedding(table: Long, tableDtype: Int, ids: Long, out: Long, positions: Int, vocab: Int, dim: Int, stream: Long) =
        check(embedding.invokeExact(ptr(table), tableDtype, ptr(ids), ptr(out), positions, vocab, dim, ptr(stream)) as Int)

    fun rmsnorm(x: Long, gain: Long, out: Long, outDtype: Int, rows: Int, n: Int, eps: Float, stream: Long) =
        check(rmsnorm.invokeExact(ptr(x), ptr(gain), ptr(out), outDtype, rows, n, eps, ptr(stream)) as Int)

    @Suppress("LongParameterList")
    fun ropeKvWrite(
        q: Long, k: Long, v: Long, positions: Long, cosTable: Long, sinTable: Long, slotMapping: Long, qOut: Long, qOutDtype: Int,
        keyCache: Long, valueCache: Long, kvDtype: Int, numTokens: Int, numHeads: Int, numKvHeads: Int, headDim: Int,
        numSlots: Int, maxPos: Int, ldQ: Int, ldK: Int, ldV: Int, stream: Long,
    ) = check(
        ropeKvWrite.invokeExact(
            ptr(q), ptr(k), ptr(v), ptr(positions), ptr(cosTable), ptr(sinTable), ptr(slotMapping), ptr(qOut), qOutDtype,
            ptr(keyCache), ptr(valueCache), kvDtype, numTokens, numHeads, numKvHeads, headDim, numSlots, maxPos, ldQ, ldK, ldV, ptr(stream),
        ) as Int,
    )

    fun swiglu(gate: Long, up: Long, ld: Int, out: Long, outDtype: Int, rows: Int, n: Int, stream: Long) =
        check(swiglu.invokeExact(ptr(gate), ptr(up), ld, ptr(out), outDtype, rows, n, ptr(stream)) as Int)

    fun argmax(logits: Long, out: Long, rows: Int, n: Int, stream: Long) =
        check(argmax.invokeExact(ptr(logits), ptr(out), rows, n, ptr(stream)) as Int)

    /** Peer-mapped memory of the tensor-parallel sum: returns (device pointer, 64-byte handle to send to the other ranks). */
    fun peerAlloc(arena: Arena, bytes: Long): Pair<Long, ByteArray> {
        val out = arena.allocate(ADDRESS)
        val handle = arena.allocate(64)
        check(peerAlloc.invokeExact(bytes, out, handle) as Int)
        return out.get(ADDRESS, 0).address() to handle.toArray(java.lang.foreign.ValueLayout.JAVA_BYTE)
    }

    fun peerOpen(arena: Arena, handle: ByteArray): Long {
        val h = arena.allocate(64)
        MemorySegment.copy(handle, 0, h, java.lang.foreign.ValueLayout.JAVA_BYTE, 0, 64)
        val out = arena.allocate(ADDRESS)
        check(peerOpen.invokeExact(h, out) as Int)
        return out.get(ADDRESS, 0).address()
    }

    fun peerClose(ptr: Long) = check(peerClose.invokeExact(ptr(ptr)) as Int)

    fun peerFree(ptr: Long) = check(peerFree.invokeExact(ptr(ptr)) as Int)

    /** In-place sum over the ranks; [bases] holds, in this process, the address of every rank's buffer. */
    fun peerAllReduceF32(arena: Arena, bases: LongArray, dataOffset: Long, flagOffset: Long, state: Long, rank: Int, count: Long, stream: Long) {
        val table = arena.allocate(ADDRESS, bases.size.toLong())
        bases.forEachIndexed { i, b -> table.setAtIndex(ADDRESS, i.toLong(), ptr(b)) }
        check(peerAllReduce.invokeExact(table, dataOffset, flagOffset, ptr(state), rank, bases.size, count, ptr(stream)) as Int)
    }

    /** The same with the following RMSNorm folded in (rows x cols at dataOffset, bf16 result at normOffset on every rank). */
    @Suppress("LongParameterList")
    fun peerAllReduceRmsnormF32(
        arena: Arena, bases: LongArray, dataOffset: Long, normOffset: Long, flagOffset: Long, state: Long, gain: Long, eps: Float,
        rank: Int, rows: Int, cols: Int, stream: Long,
    ) {
        val table = arena.allocate(ADDRESS, bases.size.toLong())
        bases.forEachIndexed { i, b -> table.setAtIndex(ADDRESS, i.toLong(), ptr(b)) }
        check(peerAllReduceNorm.invokeExact(table, dataOffset, normOffset, flagOffset, ptr(state), ptr(gain), eps, rank, bases.size, rows, cols, ptr(stream)) as Int)
    }

    /**
     * The exchange with the residual stream distributed by rows: ownRows += the ranks' partials; the RMSNorm rows go to
     * every rank as bf16, or (planes) as the int8 activation planes of the projection that reads them.
     */
    @Suppress("LongParameterList")
    fun peerReduceRmsnormRowsF32(
        arena: Arena, bases: LongArray, dataOffset: Long, normOffset: Long, flagOffset: Long, state: Long, ownRows: Long, gain: Long,
        eps: Float, rank: Int, rows: Int, cols: Int, planes: Boolean, stream: Long,
    ) {
        val table = arena.allocate(ADDRESS, bases.size.toLong())
        bases.forEachIndexed { i, b -> table.setAtIndex(ADDRESS, i.toLong(), ptr(b)) }
        check(
            peerReduceNormRows.invokeExact(
                table, dataOffset, normOffset, flagOffset, ptr(state), ptr(ownRows), ptr(gain), eps, rank, bases.size, rows, cols,
                if (planes) 1 else 0, ptr(stream),
            ) as Int,
        )
    }

    /** The one-barrier sum: out = residual + the ranks' partials at partialOffset, and the RMSNorm of it, all local. */
    @Suppress("LongParameterList")
    fun peerSumRowsF32(
        arena: Arena, bases: LongArray, partialOffset: Long, flagOffset: Long, state: Long, residual: Long, out: Long, normOut: Long,
        gain: Long, eps: Float, rank: Int, rows: Int, cols: Int, planes: Long, planesBytes: Long, stream: Long,
    ) {
        val table = arena.allocate(ADDRESS, bases.size.toLong())
        bases.forEachIndexed { i, b -> table.setAtIndex(ADDRESS, i.toLong(), ptr(b)) }
        check(
            peerSumRows.invokeExact(
                table, partialOffset, flagOffset, ptr(state), ptr(residual), ptr(out), ptr(normOut), ptr(gain), eps, rank, bases.size, rows, cols,
                ptr(planes), planesBytes, ptr(stream),
            ) as Int,
        )
    }

    /** RMSNorm with a bf16 result that also writes the int8 tensor-core projection's activation planes (GEMM_X_PLANES). */
    fun rmsnormPlanes(x: Long, gain: Long, out: Long, planes: Long, planesBytes: Long, rows: Int, n: Int, eps: Float, stream: Long) =
        check(rmsnormPlanes.invokeExact(ptr(x), ptr(gain), ptr(out), ptr(planes), planesBytes, rows, n, eps, ptr(stream)) as Int)

    /** TlalocRegisterKernels(PJRT_Api*): null on success, else the library's message. */
    fun registerKernels(pjrtApi: MemorySegment): String? {
        val err = registerKernels.invokeExact(pjrtApi) as MemorySegment
        return if (err.address() == 0L) null else err.reinterpret(4096).getString(0)
    }

    /** One typed-FFI handler by target name, as an XLA_FFI_Handler* address (0 for an unknown name). */
    fun ffiHandler(arena: Arena, target: String): Long =
        (ffiHandler.invokeExact(arena.allocateFrom(target)) as MemorySegment).address()
}
