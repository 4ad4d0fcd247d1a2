/* A minimal NVTX injection library for tests/test_tracing.py: the library under test loads it through
 * NVTX_INJECTION64_PATH and every range it opens or closes is appended to the file named by NVTX_RECORD_FILE. */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <nvtx3/nvToolsExt.h>

static void record(const char* what, const char* name) {
    const char* path = getenv("NVTX_RECORD_FILE");
    if (!path) return;
    FILE* f = fopen(path, "a");
    if (!f) return;
    fprintf(f, "%s %s\n", what, name ? name : "");
    fclose(f);
}

static int NVTX_API on_push(const char* message) {
    record("push", message);
    return 0;
}

static int NVTX_API on_pop(void) {
    record("pop", "");
    return 0;
}

typedef const void*(NVTX_API* get_export_table_t)(uint32_t);

int InitializeInjectionNvtx2(get_export_table_t get_export_table) {
    const NvtxExportTableCallbacks* cb = (const NvtxExportTableCallbacks*)get_export_table(NVTX_ETID_CALLBACKS);
    NvtxFunctionTable table = 0;
    unsigned int size = 0;
    if (!cb || !cb->GetModuleFunctionTable(NVTX_CB_MODULE_CORE, &table, &size)) return 0;
    if (size <= NVTX_CBID_CORE_RangePop) return 0;
    *table[NVTX_CBID_CORE_RangePushA] = (NvtxFunctionPointer)on_push;
    *table[NVTX_CBID_CORE_RangePop] = (NvtxFunctionPointer)on_pop;
    return 1;
}
