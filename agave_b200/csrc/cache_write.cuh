// Where a step's keys and values go, shared by the kernels that store them: the
// separate q/k norm + rotation + store kernel and the q/k/v product whose epilogue does
// the same.
#pragma once
#include "common.cuh"

// Cache addressing: position p of a sequence lives in ring row p % cap of its slot; the
// row's page comes from the slot's page table.  A token whose row a later token of the
// same step overwrites (p < len_after - cap) is not stored.
struct CacheWrite {
    void* k_pool;              // [n_pages, page, n_kv, hd] of this layer; null: nothing is stored
    void* v_pool;
    const int* page_table;     // [n_slots, max_pages]
    const int* slots;          // [B]; negative: padding entry, nothing is stored
    const int* lens;           // [B] length after this step
    const int* seq_index;      // [T] token -> batch entry
    int max_pages, page, cap;
};

// The step's values once more, transposed, for the prompt attention whose
// O += P V product wants its V operand with the keys contiguous:
// vt[g * hd + d, start(b) + p] = v[token of (b, p), g, d], where start(b) is the sum
// of the earlier sequences' lengths, each rounded up to 64; the columns between a
// sequence's end and the next multiple of 64 are zero.
struct VtWrite {
    __nv_bfloat16* vt;         // [nkv * hd, ld]; null: not wanted
    long long ld;
    const int* cu;             // [n_seq + 1] first token of each sequence
    const int* seq_index;      // [T]
};
