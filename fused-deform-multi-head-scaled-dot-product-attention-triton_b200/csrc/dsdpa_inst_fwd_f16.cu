#define DSDPA_T __half
#include "dsdpa_inst_fwd.inc"
