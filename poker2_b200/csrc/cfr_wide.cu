// The general CFR kernel for trees of up to kCfrMaxChildren (8) actions per node: fold, call, five bet sizes and
// all-in, the default bet sizes of the upstream configuration dataclass.  Same source as cfr.cu, compiled for the
// wider node bodies only (see the note at the top of that file).
#define P2B_CFR_WIDE 1
#include "cfr.cu"
