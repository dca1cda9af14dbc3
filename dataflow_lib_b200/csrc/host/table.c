/*
 * Open-addressing hash table with linear probing, fixed-size keys and values copied into
 * one flat array, and a bit vector marking free slots. Same contract as
 * als244/dataflow_lib src/table (table.h:73-102): single-threaded; insert refuses duplicate
 * keys; find returns the slot index or -1.
 *
 * Differences in mechanism: removal closes the probe sequence by shifting later entries back
 * (no tombstones, no rehash of the cluster), and a table whose load factor is >= 1 doubles
 * when it fills instead of refusing the insert while below max_size.
 */
#include "dataflow_api.h"

#include <stdlib.h>
#include <string.h>

static inline size_t slot_bytes(const Table * t) { return t->config.key_size_bytes + t->config.value_size_bytes; }
static inline uint8_t * slot_ptr(const Table * t, uint64_t i) { return (uint8_t *) t->items + i * slot_bytes(t); }
static inline bool slot_free(const Table * t, uint64_t i) { return (t->is_empty_bit_vector[i >> 6] >> (i & 63)) & 1ULL; }
static inline void mark_used(Table * t, uint64_t i) { t->is_empty_bit_vector[i >> 6] &= ~(1ULL << (i & 63)); }
static inline void mark_free(Table * t, uint64_t i) { t->is_empty_bit_vector[i >> 6] |= 1ULL << (i & 63); }

static int alloc_storage(Table * t, uint64_t size) {
	const uint64_t words = (size + 63) / 64;
	uint64_t * bits = (uint64_t *) malloc(words * sizeof(uint64_t));
	void * items = calloc(size, slot_bytes(t));
	if (!bits || !items) { free(bits); free(items); return -1; }
	memset(bits, 0xff, words * sizeof(uint64_t));
	if (size & 63) bits[words - 1] = (1ULL << (size & 63)) - 1;     /* bits past `size` read as used */
	t->is_empty_bit_vector = bits;
	t->items = items;
	t->size = size;
	return 0;
}

int init_table(Table * table, Hash_Func hash_func, uint64_t key_size_bytes, uint64_t value_size_bytes,
               uint64_t min_table_size, uint64_t max_table_size, float load_factor, float shrink_factor) {
	if (!table || !hash_func || !key_size_bytes || !min_table_size || max_table_size < min_table_size) return -1;
	table->config = (Table_Config){min_table_size, max_table_size, load_factor, shrink_factor, hash_func, key_size_bytes, value_size_bytes};
	table->cnt = 0;
	return alloc_storage(table, min_table_size);
}

void destroy_table(Table * table) {
	if (!table) return;
	free(table->is_empty_bit_vector);
	free(table->items);
	table->is_empty_bit_vector = NULL;
	table->items = NULL;
	table->size = 0;
	table->cnt = 0;
}

/* Slot holding `key`, or -1. Probing stops at the first free slot. */
static long probe(const Table * t, const void * key) {
	if (!t->items || !t->size) return -1;
	uint64_t i = t->config.hash_func((void *) key, t->size) % t->size;
	for (uint64_t n = 0; n < t->size; n++, i = (i + 1 == t->size) ? 0 : i + 1) {
		if (slot_free(t, i)) return -1;
		if (memcmp(slot_ptr(t, i), key, t->config.key_size_bytes) == 0) return (long) i;
	}
	return -1;
}

static void place(Table * t, const void * key, const void * value) {
	uint64_t i = t->config.hash_func((void *) key, t->size) % t->size;
	while (!slot_free(t, i)) i = (i + 1 == t->size) ? 0 : i + 1;
	memcpy(slot_ptr(t, i), key, t->config.key_size_bytes);
	memcpy(slot_ptr(t, i) + t->config.key_size_bytes, value, t->config.value_size_bytes);
	mark_used(t, i);
}

static int rebuild(Table * t, uint64_t new_size) {
	Table old = *t;
	if (alloc_storage(t, new_size)) { *t = old; return -1; }
	for (uint64_t i = 0; i < old.size; i++)
		if (!slot_free(&old, i)) place(t, slot_ptr(&old, i), slot_ptr(&old, i) + old.config.key_size_bytes);
	free(old.is_empty_bit_vector);
	free(old.items);
	return 0;
}

int insert_table(Table * table, void * key, void * value) {
	if (!table || !table->items || !key) return -1;
	if (probe(table, key) >= 0) {
		fprintf(stderr, "Error: key already exists in table. Cannot insert...\n");
		return -1;
	}
	const float lf = table->config.load_factor;
	const uint64_t cap = lf >= 1.0f ? table->size : (uint64_t) ((float) table->size * lf);
	if (table->cnt + 1 > cap || table->cnt == table->size) {
		if (table->size >= table->config.max_size) {
			if (table->cnt == table->size) return -1;               /* completely full at the maximum size */
		} else {
			uint64_t grown = lf > 0.0f && lf < 0.5f ? (uint64_t) ((float) table->size / lf) : table->size * 2;
			if (grown > table->config.max_size) grown = table->config.max_size;
			if (rebuild(table, grown)) return -1;
		}
	}
	place(table, key, value);
	table->cnt++;
	return 0;
}

long find_table(Table * table, void * key, bool to_copy_value, void ** ret_value) {
	if (ret_value) {
		if (to_copy_value) memset((void *) ret_value, 0, table->config.value_size_bytes);
		else *ret_value = NULL;
	}
	const long i = probe(table, key);
	if (i < 0) return -1;
	void * value = slot_ptr(table, (uint64_t) i) + table->config.key_size_bytes;
	if (ret_value) {
		/* copy mode: ret_value itself is the destination buffer (the reference's calling convention) */
		if (to_copy_value) memcpy((void *) ret_value, value, table->config.value_size_bytes);
		else *ret_value = value;
	}
	return i;
}

int remove_table(Table * table, void * key, void * ret_value) {
	long found = probe(table, key);
	if (found < 0) return -1;
	uint64_t hole = (uint64_t) found;
	if (ret_value) memcpy(ret_value, slot_ptr(table, hole) + table->config.key_size_bytes, table->config.value_size_bytes);
	/* backward-shift: pull every later entry of the run into the hole if its home slot allows it */
	uint64_t j = hole;
	for (;;) {
		j = (j + 1 == table->size) ? 0 : j + 1;
		if (j == (uint64_t) found || slot_free(table, j)) break;
		const uint64_t home = table->config.hash_func(slot_ptr(table, j), table->size) % table->size;
		const bool movable = (hole <= j) ? (home <= hole || home > j) : (home <= hole && home > j);
		if (movable) { memcpy(slot_ptr(table, hole), slot_ptr(table, j), slot_bytes(table)); hole = j; }
	}
	mark_free(table, hole);
	table->cnt--;
	const float sf = table->config.shrink_factor;
	if (sf > 0.0f && sf < 1.0f && table->size > table->config.min_size && (float) table->cnt < (float) table->size * sf) {
		uint64_t smaller = table->size / 2;
		if (smaller < table->config.min_size) smaller = table->config.min_size;
		if (smaller > table->cnt) rebuild(table, smaller);        /* failure to shrink is not an error */
	}
	return 0;
}
