/*
 * Datatype metadata and host-side conversions (als244/dataflow_lib: src/datatype/src/dataflow_datatype.c:4-90,
 * solo_conversion.c:3-156, convert_datatype.c:149-229). On the device the conversions are
 * folded into the kernels' loads and stores; the host versions exist for preparing inputs.
 *
 * fp32 -> bf16/fp16 here rounds to nearest even (what the reference's AVX-512 path and the
 * CUDA intrinsics do). The reference's scalar fall-back rounds halves up and mishandles a
 * mantissa carry in fp16; that variant is not reproduced.
 */
#include "dataflow_api.h"

#include <pthread.h>
#include <stdio.h>
#include <string.h>

size_t dataflow_sizeof_element(DataflowDatatype arr_dtype) {
	switch (arr_dtype) {
		case DATAFLOW_FP64: case DATAFLOW_UINT64: return 8;
		case DATAFLOW_FP32: case DATAFLOW_UINT32: return 4;
		case DATAFLOW_FP16: case DATAFLOW_BF16: case DATAFLOW_UINT16: return 2;
		case DATAFLOW_FP8E4M3: case DATAFLOW_FP8E5M2: case DATAFLOW_UINT8: return 1;
		case DATAFLOW_LONG: return sizeof(long);
		case DATAFLOW_INT: return sizeof(int);
		default: return 0;          /* NONE, VOID, BOOL and every *_SCALAR kind */
	}
}

char * dataflow_datatype_as_string(DataflowDatatype dtype) {
	static char * const names[] = {
		[DATAFLOW_VOID] = "VOID", [DATAFLOW_FP64] = "FP64", [DATAFLOW_FP32] = "FP32", [DATAFLOW_FP16] = "FP16",
		[DATAFLOW_BF16] = "BF16", [DATAFLOW_FP8E4M3] = "FP8E4M3", [DATAFLOW_FP8E5M2] = "FP8E5M2",
		[DATAFLOW_UINT64] = "UINT64", [DATAFLOW_UINT32] = "UINT32", [DATAFLOW_UINT16] = "UINT16",
		[DATAFLOW_UINT8] = "UINT8", [DATAFLOW_LONG] = "LONG", [DATAFLOW_INT] = "INT",
	};
	if ((int) dtype > 0 && (size_t) dtype < sizeof(names) / sizeof(names[0]) && names[dtype]) return names[dtype];
	return "UNKNOWN";
}

/* ---- scalar conversions -------------------------------------------------------------- */

float solo_bf16_to_fp32(uint16_t a) {
	uint32_t bits = (uint32_t) a << 16;
	float f;
	memcpy(&f, &bits, 4);
	return f;
}

uint16_t solo_fp32_to_bf16(float f) {
	uint32_t bits;
	memcpy(&bits, &f, 4);
	if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t) ((bits >> 16) | 0x0040u);   /* quiet NaN */
	bits += 0x7fffu + ((bits >> 16) & 1u);
	return (uint16_t) (bits >> 16);
}

float solo_fp16_to_fp32(uint16_t h) {
	const uint32_t sign = (uint32_t) (h & 0x8000u) << 16;
	uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
	if (exp == 0x1fu) bits = sign | 0x7f800000u | (man << 13);
	else if (exp) bits = sign | ((exp + 112u) << 23) | (man << 13);
	else if (!man) bits = sign;
	else {                                   /* subnormal half -> normal float */
		int shift = 0;
		while (!(man & 0x400u)) { man <<= 1; shift++; }
		bits = sign | ((uint32_t) (113 - shift) << 23) | ((man & 0x3ffu) << 13);
	}
	float f;
	memcpy(&f, &bits, 4);
	return f;
}

uint16_t solo_fp32_to_fp16(float f) {
	uint32_t bits;
	memcpy(&bits, &f, 4);
	const uint16_t sign = (uint16_t) ((bits >> 16) & 0x8000u);
	const uint32_t abs = bits & 0x7fffffffu;
	if (abs > 0x7f800000u) return sign | 0x7e00u;                 /* NaN */
	if (abs >= 0x477ff000u) return sign | 0x7c00u;                /* rounds to >= 65520 -> inf */
	if (abs < 0x33000001u) return sign;                           /* <= 2^-25 -> 0 */
	const int exp = (int) (abs >> 23) - 127;
	uint32_t man = (abs & 0x7fffffu) | 0x800000u;
	int shift;                                                    /* bits dropped from the 24-bit significand */
	uint32_t base;
	if (exp < -14) { shift = 13 + (-14 - exp); base = 0; }        /* subnormal result */
	else { shift = 13; base = (uint32_t) (exp + 15) << 10; man &= 0x7fffffu; }
	uint32_t q = man >> shift;
	const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
	if (rem > halfway || (rem == halfway && (q & 1u))) q++;       /* carries ripple into the exponent correctly */
	return sign | (uint16_t) (base + q);
}

uint16_t solo_fp16_to_bf16(uint16_t h) { return solo_fp32_to_bf16(solo_fp16_to_fp32(h)); }
uint16_t solo_bf16_to_fp16(uint16_t a) { return solo_fp32_to_fp16(solo_bf16_to_fp32(a)); }

/* ---- threaded array conversion -------------------------------------------------------- */

typedef struct {
	void * to; const void * from;
	DataflowDatatype to_dt, from_dt;
	long begin, end;
} Convert_Job;

static float load_as_fp32(const void * p, DataflowDatatype dt, long i) {
	switch (dt) {
		case DATAFLOW_FP32: return ((const float *) p)[i];
		case DATAFLOW_FP16: return solo_fp16_to_fp32(((const uint16_t *) p)[i]);
		default:            return solo_bf16_to_fp32(((const uint16_t *) p)[i]);
	}
}

/* Vector paths for the two conversions that make 16-bit inputs from fp32 and back (8 lanes of integer arithmetic, AVX2; chosen at
 * run time). They produce the scalar functions' bits: NaN lanes are patched by the scalar code. */
#if defined(__x86_64__)
#include <immintrin.h>
__attribute__((target("avx2")))
static long fp32_to_bf16_avx2(uint16_t * to, const float * from, long begin, long end) {
	long i = begin;
	const __m256i bias = _mm256_set1_epi32(0x7fff), one = _mm256_set1_epi32(1), absmask = _mm256_set1_epi32(0x7fffffff), inf = _mm256_set1_epi32(0x7f800000);
	for (; i + 8 <= end; i += 8) {
		const __m256i u = _mm256_loadu_si256((const __m256i *) (from + i));
		const __m256i nan = _mm256_cmpgt_epi32(_mm256_and_si256(u, absmask), inf);
		const __m256i r = _mm256_srli_epi32(_mm256_add_epi32(u, _mm256_add_epi32(bias, _mm256_and_si256(_mm256_srli_epi32(u, 16), one))), 16);
		const __m128i packed = _mm_packus_epi32(_mm256_castsi256_si128(r), _mm256_extracti128_si256(r, 1));
		_mm_storeu_si128((__m128i *) (to + i), packed);
		if (_mm256_movemask_epi8(nan)) for (int k = 0; k < 8; k++) to[i + k] = solo_fp32_to_bf16(from[i + k]);
	}
	return i;
}
__attribute__((target("avx2")))
static long bf16_to_fp32_avx2(float * to, const uint16_t * from, long begin, long end) {
	long i = begin;
	for (; i + 8 <= end; i += 8) {
		const __m256i w = _mm256_cvtepu16_epi32(_mm_loadu_si128((const __m128i *) (from + i)));
		_mm256_storeu_si256((__m256i *) (to + i), _mm256_slli_epi32(w, 16));
	}
	return i;
}
/* fp16 through the F16C converters (round to nearest even, subnormals handled in hardware) */
__attribute__((target("avx2,f16c")))
static long fp32_to_fp16_f16c(uint16_t * to, const float * from, long begin, long end) {
	long i = begin;
	const __m256i absmask = _mm256_set1_epi32(0x7fffffff), inf = _mm256_set1_epi32(0x7f800000);
	for (; i + 8 <= end; i += 8) {
		const __m256 v = _mm256_loadu_ps(from + i);
		const __m256i nan = _mm256_cmpgt_epi32(_mm256_and_si256(_mm256_castps_si256(v), absmask), inf);
		_mm_storeu_si128((__m128i *) (to + i), _mm256_cvtps_ph(v, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
		if (_mm256_movemask_epi8(nan)) for (int k = 0; k < 8; k++) to[i + k] = solo_fp32_to_fp16(from[i + k]);
	}
	return i;
}
__attribute__((target("avx2,f16c")))
static long fp16_to_fp32_f16c(float * to, const uint16_t * from, long begin, long end) {
	long i = begin;
	for (; i + 8 <= end; i += 8) {
		const __m128i h = _mm_loadu_si128((const __m128i *) (from + i));
		const __m128i expo = _mm_and_si128(h, _mm_set1_epi16(0x7c00)), mant = _mm_and_si128(h, _mm_set1_epi16(0x03ff));
		const int nan = _mm_movemask_epi8(_mm_andnot_si128(_mm_cmpeq_epi16(mant, _mm_setzero_si128()), _mm_cmpeq_epi16(expo, _mm_set1_epi16(0x7c00))));
		_mm256_storeu_ps(to + i, _mm256_cvtph_ps(h));
		if (nan) for (int k = 0; k < 8; k++) to[i + k] = solo_fp16_to_fp32(from[i + k]);
	}
	return i;
}
static int have_avx2(void) { static int v = -1; if (v < 0) v = __builtin_cpu_supports("avx2") ? 1 : 0; return v; }
static int have_f16c(void) { static int v = -1; if (v < 0) v = (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c")) ? 1 : 0; return v; }
#else
static int have_avx2(void) { return 0; }
#endif

static void * convert_worker(void * arg) {
	Convert_Job * job = (Convert_Job *) arg;
#if defined(__x86_64__)
	if (have_avx2()) {
		if (job->from_dt == DATAFLOW_FP32 && job->to_dt == DATAFLOW_BF16) job->begin = fp32_to_bf16_avx2((uint16_t *) job->to, (const float *) job->from, job->begin, job->end);
		else if (job->from_dt == DATAFLOW_BF16 && job->to_dt == DATAFLOW_FP32) job->begin = bf16_to_fp32_avx2((float *) job->to, (const uint16_t *) job->from, job->begin, job->end);
	}
	if (have_f16c()) {
		if (job->from_dt == DATAFLOW_FP32 && job->to_dt == DATAFLOW_FP16) job->begin = fp32_to_fp16_f16c((uint16_t *) job->to, (const float *) job->from, job->begin, job->end);
		else if (job->from_dt == DATAFLOW_FP16 && job->to_dt == DATAFLOW_FP32) job->begin = fp16_to_fp32_f16c((float *) job->to, (const uint16_t *) job->from, job->begin, job->end);
	}
#endif
	for (long i = job->begin; i < job->end; i++) {
		const float v = load_as_fp32(job->from, job->from_dt, i);
		switch (job->to_dt) {
			case DATAFLOW_FP32: ((float *) job->to)[i] = v; break;
			case DATAFLOW_FP16: ((uint16_t *) job->to)[i] = solo_fp32_to_fp16(v); break;
			default:            ((uint16_t *) job->to)[i] = solo_fp32_to_bf16(v); break;
		}
	}
	return NULL;
}

static bool convertible(DataflowDatatype dt) { return dt == DATAFLOW_FP32 || dt == DATAFLOW_FP16 || dt == DATAFLOW_BF16; }

int dataflow_convert_datatype(void * to, void * from, DataflowDatatype to_dt, DataflowDatatype from_dt, long n, int num_threads) {
	if (!convertible(to_dt) || !convertible(from_dt)) {
		fprintf(stderr, "Error: host conversion from %s to %s is not supported (fp32, fp16, bf16 only)\n",
		        dataflow_datatype_as_string(from_dt), dataflow_datatype_as_string(to_dt));
		return -1;
	}
	if (n <= 0) return 0;
	if (to_dt == from_dt) { memcpy(to, from, (size_t) n * dataflow_sizeof_element(to_dt)); return 0; }
	if (num_threads < 1) num_threads = 1;
	if (num_threads > 256) num_threads = 256;
	if ((long) num_threads > n) num_threads = (int) n;
	pthread_t threads[256];
	bool joinable[256];
	Convert_Job jobs[256];
	const long per = (n + num_threads - 1) / num_threads;
	for (int t = 0; t < num_threads; t++) {
		const long begin = t * per, end = (t + 1) * per < n ? (t + 1) * per : n;
		jobs[t] = (Convert_Job){to, from, to_dt, from_dt, begin, end};
		joinable[t] = false;
		if (begin >= end) continue;
		/* the last slice, and any slice whose thread cannot be created, runs on the caller */
		if (t < num_threads - 1 && pthread_create(&threads[t], NULL, convert_worker, &jobs[t]) == 0) joinable[t] = true;
		else convert_worker(&jobs[t]);
	}
	for (int t = 0; t < num_threads; t++) if (joinable[t]) pthread_join(threads[t], NULL);
	return 0;
}
