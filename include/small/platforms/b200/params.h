// params.h -- blocking constants of the B200 platform (contract:
// docs/Defining_Platforms.md of the reference; compare platforms/zen2/params.h:16-20).
//
// Both element types use a channel block of 16: for uint8 one pixel's block is 16 bytes,
// one row of a tensor-core core matrix; for float it is 64 bytes, one TMA swizzle row.
// W_ob has no meaning on the GPU (the pixel tile is chosen per kernel) and is kept only
// because callers read BufferT::W_ob.
#pragma once

#define SMALL_HAS_FLOAT_SUPPORT 1
#define FLOAT_W_ob 6
#define FLOAT_C_ob 16
#define FLOAT_SIMD 4
#define FLOAT_UNROLL 1
#define FLOAT_C_ib FLOAT_C_ob
#define FLOAT_NUM_FMA 1
#define FLOAT_NUM_MAX 1
#define FLOAT_NUM_LOAD 1
#define FLOAT_NUM_STORE 1

#define SMALL_HAS_QUINT8_SUPPORT 1
#define QUINT8_W_ob 2
#define QUINT8_C_ob 16
#define QUINT8_SIMD 16
#define QUINT8_UNROLL 1
#define QUINT8_C_ib QUINT8_C_ob
#define QUINT8_NUM_FMA 1
#define QUINT8_NUM_MAX 1
#define QUINT8_NUM_LOAD 1
#define QUINT8_NUM_STORE 1
