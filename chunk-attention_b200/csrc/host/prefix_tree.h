// The prefix tree of fixed-size KV chunks: shared-prefix detection on insert, reference counts,
// one private tail per live sequence, and the depth-first chunk list a decode step is planned
// from.  Pure host metadata, no device calls.
//
// Behaviour follows the reference's GPT::Attention tree maintenance
// (cpp/chunk_attn/attention.cpp:116-131,141-193,263-313,342-372); the tree-shape assertions of
// tests/test_chunk_attn_cpu.py:24-215,267-303 hold for it unchanged.
#pragma once
#include <vector>

#include "../../../include/chunk_attn_b200.h"
#include "chunk.h"

namespace ca_host {

struct NewChunk {
    Chunk* chunk;
    int token_start;  // position of the chunk's first token in the inserted sequence
    int n_tokens;
};

class PrefixTree {
  public:
    PrefixTree(int chunk_size, int64_t max_chunks, int64_t chunk_bytes, bool share_prefix);

    // Insert a sequence.  Returns its row index (its position in depth-first order of tails);
    // `created` lists the chunks whose K/V the caller must fill (an empty reserved tail is not
    // listed).
    int add_seq(const std::vector<int>& tokens, std::vector<NewChunk>& created);
    void remove_seq(int seq_idx);
    // Give every full tail an empty child; returns the new chunks.
    std::vector<Chunk*> reserve();
    // Record one new token id per sequence in its tail (the K/V rows are written on the device).
    void append_token_ids(const std::vector<int>& tokens);
    // Clone the leaf of `seq_idx` `copies` times as its next siblings (beam search); `pairs`
    // receives (source, clone) for the device copy.
    void duplicate(int seq_idx, int copies, std::vector<std::pair<Chunk*, Chunk*>>& pairs);
    // Fork row `seq_idx` into tokens.size() rows, each continuing with its own token (one beam-search
    // step): the source keeps its row and takes tokens[0], clones of its leaf follow as rows
    // seq_idx + 1 ... and take tokens[1] ....  `pairs` receives (source, clone) for the device copy,
    // `slots` the (chunk, row in chunk) token i's K/V must be written to.  Leaves that fill up get
    // their empty successor.  Nothing is changed when the pool cannot hold the result.
    void append_completion(int seq_idx, const std::vector<int>& tokens, std::vector<std::pair<Chunk*, Chunk*>>& pairs,
                           std::vector<std::pair<Chunk*, int>>& slots);
    void clear();

    std::vector<ca_chunk_info> get_chunks() const;
    Chunk* root() { return root_.get(); }
    const std::vector<Chunk*>& tails() const { return tails_; }
    int n_seqs() const { return (int)tails_.size(); }
    ChunkPool& pool() { return pool_; }
    const ChunkPool& pool() const { return pool_; }
    int chunk_size() const { return chunk_size_; }

  private:
    int chunk_size_;
    bool share_prefix_;
    ChunkPool pool_;
    std::unique_ptr<Chunk> root_;
    std::vector<Chunk*> tails_;
};

}  // namespace ca_host
