// fread / fwrite on tensor memory.
//
// The host program checkpoints by handing tensor memory straight to stdio
// (reference src/vit.c:1123-1142).  For anything larger than the stream's
// buffer the C library passes the caller's pointer to read(2) / write(2), and
// a system call on a mirror whose pages are protected (contents on the device)
// does not raise the page fault the coherence layer lives on: it just fails
// with EFAULT.  These two definitions sit in front of the C library's in the
// lookup order of any program linked against this library (the reference's
// link line puts it before libc); they bring the affected mirrors up to date
// on the host side first and then call the real function.  Memory that is not
// tensor memory is recognised by an address-range check and passed through.
//
// VITB200_NO_STDIO_HOOKS=1 turns the preparation off (the functions still
// forward), for hosts that call vitb200_make_host_coherent themselves.
#include "coherence.h"

#include <cstdio>
#include <cstdlib>
#include <dlfcn.h>

namespace {

typedef size_t (*ReadFunction)(void *, size_t, size_t, FILE *);
typedef size_t (*WriteFunction)(const void *, size_t, size_t, FILE *);

bool hooks_enabled() {
    static const bool enabled = [] {
        const char *text = getenv("VITB200_NO_STDIO_HOOKS");
        return !(text && text[0] == '1');
    }();
    return enabled;
}

}  // namespace

extern "C" size_t fwrite(const void *pointer, size_t size, size_t count,
                         FILE *stream) {
    static const WriteFunction real =
        reinterpret_cast<WriteFunction>(dlsym(RTLD_NEXT, "fwrite"));
    if (hooks_enabled()) {
        vitb200::coherent_prepare_host_io(pointer, size * count, false);
    }
    return real ? real(pointer, size, count, stream) : 0;
}

extern "C" size_t fread(void *pointer, size_t size, size_t count, FILE *stream) {
    static const ReadFunction real =
        reinterpret_cast<ReadFunction>(dlsym(RTLD_NEXT, "fread"));
    if (hooks_enabled()) {
        vitb200::coherent_prepare_host_io(pointer, size * count, true);
    }
    return real ? real(pointer, size, count, stream) : 0;
}
