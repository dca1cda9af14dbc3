/*
 * Op fingerprints. The registry key of an op is the SHA-256 digest of its 388-byte skeleton
 * header (als244/dataflow_lib: src/fingerprint/src/fingerprint.c:114-138 calls OpenSSL for
 * this). SHA-256 (FIPS 180-4) is implemented here so that the library carries no libcrypto
 * dependency; the digests are identical.
 */
#include "dataflow_api.h"

#include <stdio.h>
#include <string.h>

static const uint32_t K256[64] = {
	0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
	0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
	0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
	0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
	0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
	0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
	0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
	0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2
};

static inline uint32_t rotr32(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

static void sha256_block(uint32_t h[8], const uint8_t blk[64]) {
	uint32_t w[64];
	for (int t = 0; t < 16; t++)
		w[t] = ((uint32_t) blk[4 * t] << 24) | ((uint32_t) blk[4 * t + 1] << 16) | ((uint32_t) blk[4 * t + 2] << 8) | blk[4 * t + 3];
	for (int t = 16; t < 64; t++) {
		uint32_t s0 = rotr32(w[t - 15], 7) ^ rotr32(w[t - 15], 18) ^ (w[t - 15] >> 3);
		uint32_t s1 = rotr32(w[t - 2], 17) ^ rotr32(w[t - 2], 19) ^ (w[t - 2] >> 10);
		w[t] = w[t - 16] + s0 + w[t - 7] + s1;
	}
	uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], k = h[7];
	for (int t = 0; t < 64; t++) {
		uint32_t t1 = k + (rotr32(e, 6) ^ rotr32(e, 11) ^ rotr32(e, 25)) + ((e & f) ^ (~e & g)) + K256[t] + w[t];
		uint32_t t2 = (rotr32(a, 2) ^ rotr32(a, 13) ^ rotr32(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
		k = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
	}
	h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += k;
}

void dataflow_sha256(const void * data, uint64_t num_bytes, uint8_t digest[32]) {
	uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
	const uint8_t * p = (const uint8_t *) data;
	uint64_t left = num_bytes;
	while (left >= 64) { sha256_block(h, p); p += 64; left -= 64; }
	uint8_t tail[128];
	memset(tail, 0, sizeof(tail));
	memcpy(tail, p, left);
	tail[left] = 0x80;
	const int tail_len = left < 56 ? 64 : 128;
	const uint64_t bits = num_bytes * 8;
	for (int i = 0; i < 8; i++) tail[tail_len - 1 - i] = (uint8_t) (bits >> (8 * i));
	sha256_block(h, tail);
	if (tail_len == 128) sha256_block(h, tail + 64);
	for (int i = 0; i < 8; i++) {
		digest[4 * i] = (uint8_t) (h[i] >> 24); digest[4 * i + 1] = (uint8_t) (h[i] >> 16);
		digest[4 * i + 2] = (uint8_t) (h[i] >> 8); digest[4 * i + 3] = (uint8_t) h[i];
	}
}

uint8_t get_fingerprint_num_bytes(FingerprintType fingerprint_type) {
	switch (fingerprint_type) {
		case SHA256_HASH: return 32;
		case SHA512_HASH: return 64;
		case SHA1_HASH: return 20;
		case MD5_HASH: return 16;
		case BLAKE3_HASH: return 32;
		default: return 0;
	}
}

char * get_fingerprint_type_name(FingerprintType fingerprint_type) {
	switch (fingerprint_type) {
		case SHA256_HASH: return "SHA256";
		case SHA512_HASH: return "SHA512";
		case SHA1_HASH: return "SHA1";
		case MD5_HASH: return "MD5";
		case BLAKE3_HASH: return "BLAKE3";
		default: return "UNKNOWN";
	}
}

/* Only SHA-256 is used by the op registry; the other digest kinds of the reference's enum are
 * reported as unsupported instead of being silently substituted. */
void do_fingerprinting(void * data, uint64_t num_bytes, uint8_t * ret_fingerprint, FingerprintType fingerprint_type) {
	if (fingerprint_type == SHA256_HASH) {
		dataflow_sha256(data, num_bytes, ret_fingerprint);
		return;
	}
	fprintf(stderr, "Error: fingerprint type %s is not supported (only SHA256)\n", get_fingerprint_type_name(fingerprint_type));
}

uint64_t fingerprint_to_least_sig64(uint8_t * fingerprint, int fingerprint_num_bytes) {
	uint64_t v = 0;
	for (int i = fingerprint_num_bytes - 8; i < fingerprint_num_bytes; i++) v = (v << 8) | fingerprint[i];
	return v;
}

void print_hex(uint8_t * fingerprint, int num_bytes) {
	for (int i = 0; i < num_bytes; i++) printf("%02x", fingerprint[i]);
	printf("\n");
}

void print_sha256(uint8_t * fingerprint) { print_hex(fingerprint, 32); }
