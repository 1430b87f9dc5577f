#define FA_INST_T __nv_bfloat16
#define FA_INST_NAME launch_decode_128_bf16
#include "decode_inst.inc"
