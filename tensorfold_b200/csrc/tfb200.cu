// The whole library as one translation unit (the kernels share one device status word and inline helpers).
#include "api.cu"
#include "routing.cu"
#include "pack.cu"
#include "experts_decode.cu"
#include "experts_prefill.cu"
#include "exl3.cu"
#include "peer.cu"
