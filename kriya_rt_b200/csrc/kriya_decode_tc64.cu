// The tensor-core decode kernel with 64-token tiles and two resident CTAs per SM: the same source as
// kriya_decode_tc.cu, compiled into namespace kriya::t64 with launchers named *_t64.  Its rings fit twice into an
// SM, so one CTA streams while its neighbour starts up, hands over partial states or merges; it is the faster kernel when
// every CTA has a long stream ahead of it (long contexts), the 128-token kernel when a launch is short.
#define KRIYA_TC_TILE64 1
#include "kriya_decode_tc.cu"
