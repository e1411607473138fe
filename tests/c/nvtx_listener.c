/* Test-only NVTX v3 injection library: an application that uses the header-only NVTX stubs loads the library named
 * by NVTX_INJECTION64_PATH on its first NVTX call and hands it the callback tables. This listener appends one line per
 * domain creation and per pushed / popped range to the file named by DUQ4_NVTX_LOG. */
#include <nvtx3/nvToolsExt.h>
#include <stdio.h>
#include <stdlib.h>

static void logline(const char *what, const char *name) {
    const char *path = getenv("DUQ4_NVTX_LOG");
    if (!path) return;
    FILE *f = fopen(path, "a");
    if (!f) return;
    fprintf(f, "%s %s\n", what, name ? name : "");
    fclose(f);
}

static nvtxDomainHandle_t NVTX_API on_domain_create(const char *name) {
    logline("domain", name);
    return (nvtxDomainHandle_t)0x1;
}
static int NVTX_API on_push(nvtxDomainHandle_t d, const nvtxEventAttributes_t *a) {
    (void)d;
    logline("push", a && a->messageType == NVTX_MESSAGE_TYPE_ASCII ? a->message.ascii : "?");
    return 0;
}
static int NVTX_API on_pop(nvtxDomainHandle_t d) {
    (void)d;
    logline("pop", "");
    return 0;
}

int InitializeInjectionNvtx2(NvtxGetExportTableFunc_t get_table) {
    const NvtxExportTableCallbacks *cb = (const NvtxExportTableCallbacks *)get_table(NVTX_ETID_CALLBACKS);
    NvtxFunctionTable table = 0;
    unsigned int size = 0;
    if (!cb || !cb->GetModuleFunctionTable(NVTX_CB_MODULE_CORE2, &table, &size)) return 0;
    if (size <= NVTX_CBID_CORE2_DomainCreateA) return 0;
    *table[NVTX_CBID_CORE2_DomainCreateA] = (NvtxFunctionPointer)on_domain_create;
    *table[NVTX_CBID_CORE2_DomainRangePushEx] = (NvtxFunctionPointer)on_push;
    *table[NVTX_CBID_CORE2_DomainRangePop] = (NvtxFunctionPointer)on_pop;
    return 1;
}
