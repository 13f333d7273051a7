/* A minimal NVTX tool for tests/test_profiling.py: loaded through NVTX_INJECTION64_PATH, it appends every
 * nvtxRangePushA / nvtxRangePop to the file named by KXC_NVTX_PROBE_LOG. Uses only NVTX's public injection interface
 * (nvtx3/nvtxDetail/nvtxTypes.h). */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <nvtx3/nvToolsExt.h>

static FILE* g_log;

static int NVTX_API probe_push(const char* message) {
    if (g_log) {
        fprintf(g_log, "push %s\n", message ? message : "");
        fflush(g_log);
    }
    return 0;
}

static int NVTX_API probe_pop(void) {
    if (g_log) {
        fprintf(g_log, "pop\n");
        fflush(g_log);
    }
    return 0;
}

int InitializeInjectionNvtx2(NvtxGetExportTableFunc_t get_export_table) {
    const char* path = getenv("KXC_NVTX_PROBE_LOG");
    const NvtxExportTableCallbacks* callbacks;
    NvtxFunctionTable table = 0;
    unsigned int size = 0;
    if (!path || !get_export_table) return 0;
    callbacks = (const NvtxExportTableCallbacks*)get_export_table(NVTX_ETID_CALLBACKS);
    if (!callbacks || !callbacks->GetModuleFunctionTable(NVTX_CB_MODULE_CORE, &table, &size)) return 0;
    if (size <= NVTX_CBID_CORE_RangePop) return 0;
    g_log = fopen(path, "a");
    if (!g_log) return 0;
    *table[NVTX_CBID_CORE_RangePushA] = (NvtxFunctionPointer)probe_push;
    *table[NVTX_CBID_CORE_RangePop] = (NvtxFunctionPointer)probe_pop;
    return 1;
}
