// small.h -- top-level include of the B200 platform build.
//
// The reference's drivers say `#include <small.h>`; with this repository's include/
// directory ahead of the reference's on the include path they get this file.  It pulls the
// platform (params, device-resident buffers, C ABI), the reference's host-side helpers
// (padding math, packing, the interface declarations -- all taken from the reference tree
// unchanged) and then THIS repository's definitions of the layer functions, which forward
// to libsmall_b200.so instead of instantiating the CPU loop nest.
#pragma once

#define SMALL_MAJOR_VERSION 1
#define SMALL_MINOR_VERSION 0
#define SMALL_SUB_VERSON 0
#define SMALL_PLATFORM_B200 1

#include <omp.h>   // the reference's <small.h> brings it in (abstract_layer.hpp:18); its demos rely on that
#include <stdint.h>

#include <params.h>      // include/small/platforms/b200
#include <Buffer.hpp>    // include/small/platforms/b200
#include <intrinsics.h>  // include/small/platforms/b200

#include <small/utils.hpp>      // reference tree
#include <small/buffers.hpp>    // reference tree
#include <small/interface.hpp>  // reference tree (declarations)

#include <small/interface_abstract.hpp>           // this repository
#include <small/interface_abstract_1D.hpp>        // this repository
#include <small/fused_interface_abstract.hpp>     // this repository
#include <small/fused_interface_abstract_1D.hpp>  // this repository
