// Status codes shared by host and device code (plain C).
#pragma once

#define NG_OK 0
#define NG_ERR_INVALID_ARG (-1)
#define NG_ERR_UNSUPPORTED (-2)
#define NG_ERR_CUDA (-3)
#define NG_ERR_NVRTC (-4)
#define NG_ERR_NCCL (-5)
#define NG_ERR_TIMEOUT (-6)
#define NG_ERR_NOT_INITIALIZED (-7)
#define NG_ERR_TOO_LARGE (-8)

// Device-side wait sites, written to the status word when a bounded wait gives up.
#define NG_DEV_TIMEOUT_PRODUCER 101
#define NG_DEV_TIMEOUT_MMA 102
#define NG_DEV_TIMEOUT_EPILOGUE 103
#define NG_DEV_TIMEOUT_ACC 104
#define NG_DEV_TIMEOUT_TEST 105
#define NG_DEV_TIMEOUT_PEER 106   /* a peer GPU's flag in the peer-memory gradient sum */
