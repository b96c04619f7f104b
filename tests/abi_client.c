/* A plain C99 client of the library: includes the public header, binds every call it uses with
 * dlopen/dlsym the way a foreign-function layer would, and exercises the host-side argument
 * checks (no GPU needed).  Prints "abi client ok" and exits 0 when everything behaves as the
 * header says.  Built and run by tests/test_abi_symbols.py. */
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include "ivab.h"

#define BIND(name)                                                        \
    name##_fn name##_p;                                                   \
    *(void**)(&name##_p) = dlsym(lib, #name);                             \
    if (!name##_p) { fprintf(stderr, "missing symbol %s\n", #name); return 2; }

typedef int (*ivab_version_fn)(void);
typedef const char* (*ivab_last_error_fn)(void);
typedef int (*ivab_decode_workspace_bytes_fn)(int64_t, int64_t, int64_t, int64_t, size_t*);
typedef int (*ivab_paged_append_fn)(const void*, const void*, int64_t, int64_t, const int64_t*, void*, void*, int64_t,
                                    int64_t, int, int64_t, int64_t, int64_t, int64_t, int64_t, int32_t*, void*);
typedef int (*ivab_paged_decode_attn_fn)(const void*, int64_t, int64_t, const void*, const void*, int64_t, int64_t,
                                         const int32_t*, int64_t, const int32_t*, const int32_t*, int64_t, void*,
                                         int64_t, int64_t, float*, int, int, int64_t, int64_t, int64_t, int64_t, int64_t,
                                         int64_t, int64_t, float, void*, size_t, void*);

int main(int argc, char** argv) {
    if (argc < 2) { fprintf(stderr, "usage: %s /path/to/libivab.so\n", argv[0]); return 2; }
    void* lib = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
    if (!lib) { fprintf(stderr, "dlopen: %s\n", dlerror()); return 2; }
    BIND(ivab_version)
    BIND(ivab_last_error)
    BIND(ivab_decode_workspace_bytes)
    BIND(ivab_paged_append)
    BIND(ivab_paged_decode_attn)

    /* the prototypes in the header and the function-pointer types above must agree */
    /* (unevaluated: a mismatch is a compile-time diagnostic, and nothing here needs the linker) */
    (void)sizeof(ivab_paged_append_p == &ivab_paged_append);
    (void)sizeof(ivab_paged_decode_attn_p == &ivab_paged_decode_attn);
    (void)sizeof(ivab_decode_workspace_bytes_p == &ivab_decode_workspace_bytes);

    if (ivab_version_p() < 110) { fprintf(stderr, "version %d\n", ivab_version_p()); return 1; }

    size_t bytes = 0;
    if (ivab_decode_workspace_bytes_p(64, 32, 32, 128, &bytes) != IVAB_OK || bytes == 0) return 1;
    if (ivab_decode_workspace_bytes_p(64, 32, 5, 128, &bytes) != IVAB_ERR_INVALID) return 1;     /* 32 % 5 != 0 */
    if (ivab_decode_workspace_bytes_p(64, 32, 8, 128, NULL) != IVAB_ERR_INVALID) return 1;

    /* empty work is a no-op that succeeds without touching any pointer */
    if (ivab_paged_append_p(NULL, NULL, 0, 0, NULL, NULL, NULL, 0, 0, IVAB_BF16, 0, 32, 128, 16, 8, NULL, NULL) != IVAB_OK)
        return 1;
    /* null pointers with work to do: an error code and a message, never a crash */
    if (ivab_paged_append_p(NULL, NULL, 4096, 128, NULL, NULL, NULL, 1 << 20, 2048, IVAB_BF16, 4, 32, 128, 16, 8, NULL,
                            NULL) != IVAB_ERR_INVALID)
        return 1;
    if (strstr(ivab_last_error_p(), "null") == NULL) { fprintf(stderr, "message: %s\n", ivab_last_error_p()); return 1; }
    /* unknown dtype */
    if (ivab_paged_append_p(NULL, NULL, 4096, 128, NULL, NULL, NULL, 1 << 20, 2048, 42, 4, 32, 128, 16, 8, NULL, NULL) !=
        IVAB_ERR_INVALID)
        return 1;
    /* decode: page size other than 16 is refused before anything is launched */
    {
        int dummy;
        int rc = ivab_paged_decode_attn_p(&dummy, 4096, 128, &dummy, &dummy, 1 << 20, 4096, (const int32_t*)&dummy, 8,
                                          (const int32_t*)&dummy, NULL, 0, &dummy, 4096, 128, NULL, IVAB_BF16, IVAB_BF16, 1,
                                          32, 8, 128, 32, 8, 8, 0.088f, &dummy, 1 << 20, NULL);
        if (rc != IVAB_ERR_UNSUPPORTED || strstr(ivab_last_error_p(), "page_size") == NULL) {
            fprintf(stderr, "decode rc %d: %s\n", rc, ivab_last_error_p());
            return 1;
        }
    }
    puts("abi client ok");
    dlclose(lib);
    return 0;
}
