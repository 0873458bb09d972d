#define DSDPA_T __nv_bfloat16
#include "dsdpa_inst_bwd.inc"
