// Build recipe only (test infrastructure): the reference engine's own CUDA
// sources for the quantized product, compiled from where they lie (the
// Makefile passes their directory with -I) as one program, in the order and
// with the one definition its device compiles them with at start-up
// (gpu/cuda/mod.rs:85-106, 742-745).  Nothing of those sources is kept in
// this repository; the result is a cubin under oracle/_ref/.
#define TILE_STAGES 3
#include "prelude.cu"
#include "to_f16.cu"
#include "matmul_rows.cu"
#include "matmul_tile.cu"
