// Weak definitions of every THNN_Cuda<Op>_<method> and THNN_CudaDouble<Op>_<method> symbol of the
// reference header, so that the FFI binding's lookup of all 324 names succeeds.  The entry points this
// library implements are strong definitions in thnn.cu and win at link time; the rest only report
// "not implemented" through the state's error hook.
// (the header with the real prototypes is deliberately not included: the stubs take only the state)
struct THCState;

extern "C" void thcunn_b200_not_implemented(THCState *state, const char *name);

#define STUB(TYPE, NAME)                                                                                       \
    extern "C" __attribute__((visibility("default"), weak)) void THNN_##TYPE##NAME(THCState *state)           \
    {                                                                                                          \
        thcunn_b200_not_implemented(state, "THNN_" #TYPE #NAME);                                               \
    }
#define X(NAME) STUB(Cuda, NAME) STUB(CudaDouble, NAME)
#include "thnn_names.inc"
#undef X
