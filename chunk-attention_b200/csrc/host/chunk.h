// Prefix-tree node and the fixed pool of nodes (host bookkeeping only: K/V live in the device
// pool, addressed by Chunk::id).
//
// Mirrors the observable behaviour of the reference's GPT::Chunk (cpp/chunk_attn/chunk.h:9-65)
// and GPT::ChunkAllocator (cpp/chunk_attn/chunk_allocator.h:10-43): node addresses are stable
// for the life of the pool (Python compares nodes by identity), a freed node is reset and
// recycled, the lowest free slot is handed out first, exhaustion throws
// "ChunkAllocator: capacity reached".
#pragma once
#include <cstdint>
#include <memory>
#include <set>
#include <string>
#include <vector>

namespace ca_host {

class Chunk {
  public:
    Chunk(int id, int capacity) : n_seqs(1), parent(nullptr), id(id), capacity_(capacity) {
        tokens.reserve(capacity > 0 ? capacity : 0);
    }
    Chunk(const Chunk&) = delete;
    Chunk& operator=(const Chunk&) = delete;

    int capacity() const { return capacity_; }
    int n_tokens() const { return (int)tokens.size(); }
    bool full() const { return (int)tokens.size() == capacity_; }
    // true when this chunk holds exactly ids[start:end)
    bool equal(const std::vector<int>& ids, int start, int end) const;
    void append_tokens(const std::vector<int>& ids, int start, int end);
    Chunk* add_child(Chunk* child);
    Chunk* insert_child(int idx, Chunk* child);
    void reset();
    std::string to_string(bool brief = false) const;

    std::vector<int> tokens;
    std::vector<Chunk*> children;  // non-owning; the pool owns every node
    int n_seqs;
    Chunk* parent;
    const int id;  // slot in the device pool; -1 for the root

  private:
    int capacity_;
};

class ChunkPool {
  public:
    ChunkPool(int64_t max_chunks, int chunk_size, int64_t chunk_bytes);
    Chunk* allocate();
    void free(Chunk* chunk);
    int64_t max_chunks() const { return (int64_t)chunks_.size(); }
    int64_t in_use() const { return (int64_t)chunks_.size() - (int64_t)free_.size(); }
    int64_t peak_memory_allocated() const { return peak_bytes_; }

  private:
    std::vector<std::unique_ptr<Chunk>> chunks_;
    std::set<int> free_;
    int64_t chunk_bytes_;
    int64_t peak_bytes_ = 0;
};

}  // namespace ca_host
