#include "chunk.h"

#include <stdexcept>

namespace ca_host {

bool Chunk::equal(const std::vector<int>& ids, int start, int end) const {
    const int n = end - start;
    if (n_tokens() != n || end > (int)ids.size()) return false;
    for (int i = 0; i < n; i++)
        if (tokens[i] != ids[start + i]) return false;
    return true;
}

void Chunk::append_tokens(const std::vector<int>& ids, int start, int end) {
    if (end - start > capacity_ - n_tokens()) throw std::runtime_error("no enough space in Chunk");
    tokens.insert(tokens.end(), ids.begin() + start, ids.begin() + end);
}

Chunk* Chunk::add_child(Chunk* child) {
    children.push_back(child);
    child->parent = this;
    return child;
}

Chunk* Chunk::insert_child(int idx, Chunk* child) {
    children.insert(children.begin() + idx, child);
    child->parent = this;
    return child;
}

void Chunk::reset() {
    tokens.clear();
    children.clear();
    n_seqs = 1;
    parent = nullptr;
}

std::string Chunk::to_string(bool brief) const {
    std::string s = std::to_string(n_seqs) + ": [";
    if (brief && tokens.size() > 3) {
        s += std::to_string(tokens.front()) + ",...," + std::to_string(tokens.back());
    } else {
        for (size_t i = 0; i < tokens.size(); i++) {
            if (i) s += ",";
            s += std::to_string(tokens[i]);
        }
    }
    return s + "]";
}

ChunkPool::ChunkPool(int64_t max_chunks, int chunk_size, int64_t chunk_bytes) : chunk_bytes_(chunk_bytes) {
    chunks_.reserve(max_chunks);
    for (int64_t i = 0; i < max_chunks; i++) {
        chunks_.emplace_back(new Chunk((int)i, chunk_size));
        free_.insert(free_.end(), (int)i);
    }
}

Chunk* ChunkPool::allocate() {
    if (free_.empty()) throw std::runtime_error("ChunkAllocator: capacity reached");
    const int id = *free_.begin();
    free_.erase(free_.begin());
    const int64_t used = in_use() * chunk_bytes_;
    if (used > peak_bytes_) peak_bytes_ = used;
    return chunks_[id].get();
}

void ChunkPool::free(Chunk* chunk) {
    if (free_.count(chunk->id)) throw std::runtime_error("free is called, but chunk is in free list");
    chunk->reset();
    free_.insert(chunk->id);
}

}  // namespace ca_host
