// Stand-in for <hip/hip_fp16.h> so that the reference's host-only headers compile with g++.
// The reference uses it for the __half type name and the __host__/__device__ annotations only
// (datatype.hpp:2-4); nothing here is executed.
#pragma once
#ifndef __host__
#define __host__
#endif
#ifndef __device__
#define __device__
#endif
struct __half { unsigned short x; };
