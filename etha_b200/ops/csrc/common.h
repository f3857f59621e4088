// Shared by the translation units of libetha_b200_cuda: one per-thread error message buffer.
#pragma once
#define ETHA_ERR_LEN 512
#ifdef __cplusplus
extern "C" {
#endif
char* etha_err_buf(void);
#ifdef __cplusplus
}
#endif
