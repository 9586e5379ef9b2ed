/* Stand-in for Apple's CommonCrypto digest header, for compiling the reference's portable C++ on
 * Linux: only the names runtime/sha256.hpp mentions.  Nothing built here hashes anything, so the
 * three functions are declared and never defined.  TEST INFRASTRUCTURE ONLY. */
#ifndef GF_SHIM_COMMON_DIGEST_H
#define GF_SHIM_COMMON_DIGEST_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef uint32_t CC_LONG;
typedef struct CC_SHA256state_st { uint32_t count[2]; uint32_t hash[8]; uint32_t wbuf[16]; } CC_SHA256_CTX;
#define CC_SHA256_DIGEST_LENGTH 32
int CC_SHA256_Init(CC_SHA256_CTX* c);
int CC_SHA256_Update(CC_SHA256_CTX* c, const void* data, CC_LONG len);
int CC_SHA256_Final(unsigned char* md, CC_SHA256_CTX* c);
#ifdef __cplusplus
}
#endif
#endif
