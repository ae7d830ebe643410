// NOT COMPILED: no JDK, Kotlin compiler or Gradle exists in the image this repository was built in.
// Written against runtime-pjrt/src/jvmMain/kotlin/io/tlaloc/runtime/pjrt/ffm/PjrtFfiRegistry.kt:192-204 and
// runtime-pjrt/.../kptx/KptxPagedAttention.kt:57-110 of the reference.
package io.tlaloc.runtime.pjrt

import io.tlaloc.runtime.pjrt.ffm.PjrtFfiRegistry
import java.nio.file.Files
import java.nio.file.Path

/**
 * Registration of the B200 kernels with a PJRT GPU plugin, the counterpart of `KptxPagedAttention.register` for a
 * library of prebuilt kernels: one native call registers every typed-FFI target the library serves.  Call it once per
 * plugin per process, BEFORE compiling a program that names one of [TARGETS] (the plugin's FFI registry is
 * process-global and permanent, PjrtFfiRegistry.kt:27-32).
 */
object B200Kernels {
    /** The custom-call targets libtlaloc_kernels.so registers; the first keeps the reference handler's wire format. */
    val TARGETS: List<String> = listOf("tlaloc_paged_attention", "tlaloc_int8_gemm", "tlaloc_kv_cache_write")

    /** `$TLALOC_KERNELS_LIBRARY`, else libtlaloc_kernels.so beside the backend (triton/backend/pjrt_runtime.cc:139-164). */
    fun defaultLibrary(backendDir: Path): Path =
        System.getenv("TLALOC_KERNELS_LIBRARY")?.let { Path.of(it) } ?: backendDir.resolve("libtlaloc_kernels.so")

    /**
     * Loads [library] and calls its `TlalocRegisterKernels(const PJRT_Api*)` with [pluginPath]'s API.  Throws
     * IllegalStateException with the library's message when the plugin has no GPU custom-call extension or a name is
     * already taken (for example by the reference's own libtlaloc_kernels.so: only one library can own
     * `tlaloc_paged_attention` in a process).
     */
    fun register(pluginPath: Path, library: Path) {
        require(Files.isRegularFile(library)) { "$library: no such file (build it with `python -m tlaloc_b200.build`)" }
        PjrtFfiRegistry.registerNativeLibrary(pluginPath, library, symbol = "TlalocRegisterKernels")
    }
}
