#include "prefix_tree.h"

#include <algorithm>
#include <stdexcept>

namespace ca_host {

PrefixTree::PrefixTree(int chunk_size, int64_t max_chunks, int64_t chunk_bytes, bool share_prefix)
  : chunk_size_(chunk_size), share_prefix_(share_prefix), pool_(max_chunks, chunk_size, chunk_bytes),
    root_(new Chunk(-1, 0)) {
    root_->n_seqs = 0;
}

int PrefixTree::add_seq(const std::vector<int>& tokens, std::vector<NewChunk>& created) {
    created.clear();
    const int total = (int)tokens.size();

    // Pass 1, read-only: walk down while a whole chunk of ids matches a NON-LEAF child (leaves stay
    // private to their sequence).  The row index is the number of sequences under the earlier
    // siblings passed on the way.
    std::vector<Chunk*> matched;
    int seq_idx = 0, start = 0;
    Chunk* prev = root_.get();
    if (share_prefix_) {
        while (start < total) {
            start += prev->n_tokens();
            Chunk* next = nullptr;
            for (Chunk* child : prev->children) {
                if (!child->children.empty() && child->equal(tokens, start, start + child->n_tokens())) {
                    next = child;
                    break;
                }
                seq_idx += child->n_seqs;
            }
            if (!next) break;
            matched.push_back(next);
            prev = next;
        }
    } else {
        // nothing is shared: the new sequence hangs off the root after every existing one.  (The
        // reference inserts row 0 here while appending the chunks as the LAST child of the root,
        // which leaves its row order and its tree order inconsistent; this keeps them equal.)
        seq_idx = root_->n_seqs;
    }
    start = std::min(start, total);
    const int rest = total - start;
    // a full last chunk may be matched by later sequences, so it cannot be the tail: it gets an
    // empty child.  With nothing left to store, the last matched node (always full) or the root is
    // in that position.
    const bool needs_empty_tail = rest > 0 ? (rest % chunk_size_ == 0) : true;
    const int need = (rest + chunk_size_ - 1) / chunk_size_ + (needs_empty_tail ? 1 : 0);
    if (pool_.max_chunks() - pool_.in_use() < need) throw std::runtime_error("ChunkAllocator: capacity reached");

    // Pass 2: mutate.  Cannot fail any more.
    root_->n_seqs += 1;
    for (Chunk* m : matched) m->n_seqs += 1;
    for (; start < total; start += chunk_size_) {
        const int end = std::min(start + chunk_size_, total);
        Chunk* child = pool_.allocate();
        child->append_tokens(tokens, start, end);
        created.push_back(NewChunk{child, start, end - start});
        prev = prev->add_child(child);
    }
    if (needs_empty_tail) prev = prev->add_child(pool_.allocate());
    tails_.insert(tails_.begin() + seq_idx, prev);
    return seq_idx;
}

void PrefixTree::remove_seq(int seq_idx) {
    if (seq_idx < 0 || seq_idx >= (int)tails_.size()) throw std::runtime_error("seq_idx out of range");
    Chunk* node = tails_[seq_idx];
    while (node != nullptr) {
        node->n_seqs -= 1;
        Chunk* parent = node->parent;
        if (node->n_seqs <= 0 && parent != nullptr) {
            parent->children.erase(std::remove(parent->children.begin(), parent->children.end(), node),
                                   parent->children.end());
            pool_.free(node);
        }
        node = parent;
    }
    tails_.erase(tails_.begin() + seq_idx);
}

std::vector<Chunk*> PrefixTree::reserve() {
    std::vector<Chunk*> fresh;
    int need = 0;
    for (Chunk* tail : tails_) need += tail->full() ? 1 : 0;
    if (pool_.max_chunks() - pool_.in_use() < need) throw std::runtime_error("ChunkAllocator: capacity reached");
    for (size_t i = 0; i < tails_.size(); i++) {
        if (tails_[i]->full()) {
            Chunk* child = pool_.allocate();
            fresh.push_back(child);
            tails_[i] = tails_[i]->add_child(child);
        }
    }
    return fresh;
}

void PrefixTree::append_token_ids(const std::vector<int>& tokens) {
    for (size_t i = 0; i < tails_.size(); i++) tails_[i]->append_tokens(tokens, (int)i, (int)i + 1);
}

void PrefixTree::duplicate(int seq_idx, int copies, std::vector<std::pair<Chunk*, Chunk*>>& pairs) {
    pairs.clear();
    if (copies < 1) return;
    if (seq_idx < 0 || seq_idx >= (int)tails_.size()) throw std::runtime_error("seq_idx out of range");
    if (pool_.max_chunks() - pool_.in_use() < copies) throw std::runtime_error("ChunkAllocator: capacity reached");
    Chunk* leaf = tails_[seq_idx];
    for (Chunk* node = leaf->parent; node != nullptr; node = node->parent) node->n_seqs += copies;
    Chunk* parent = leaf->parent;
    const int pos = (int)(std::find(parent->children.begin(), parent->children.end(), leaf) - parent->children.begin()) + 1;
    for (int c = 0; c < copies; c++) {
        Chunk* clone = pool_.allocate();
        clone->tokens = leaf->tokens;
        parent->insert_child(pos + c, clone);
        // the clones are the rows right after the source row in depth-first order
        tails_.insert(tails_.begin() + seq_idx + 1 + c, clone);
        pairs.emplace_back(leaf, clone);
    }
}

void PrefixTree::append_completion(int seq_idx, const std::vector<int>& tokens,
                                   std::vector<std::pair<Chunk*, Chunk*>>& pairs,
                                   std::vector<std::pair<Chunk*, int>>& slots) {
    pairs.clear();
    slots.clear();
    if (seq_idx < 0 || seq_idx >= (int)tails_.size()) throw std::runtime_error("seq_idx out of range");
    if (tokens.empty()) throw std::runtime_error("append_completion: at least one token is required");
    const int n = (int)tokens.size();
    // chunks needed before anything is touched: successors of tails that are full now, the clones,
    // and successors of the forked leaves if this token fills them
    int need = n - 1;
    for (Chunk* tail : tails_) need += tail->full() ? 1 : 0;
    const Chunk* leaf = tails_[seq_idx];
    const int fill = leaf->full() ? 0 : leaf->n_tokens();
    if (fill + 1 == chunk_size_) need += n;
    if (pool_.max_chunks() - pool_.in_use() < need) throw std::runtime_error("ChunkAllocator: capacity reached");
    reserve();
    duplicate(seq_idx, n - 1, pairs);
    for (int i = 0; i < n; i++) {
        Chunk* tail = tails_[seq_idx + i];
        slots.emplace_back(tail, tail->n_tokens());
        tail->append_tokens(tokens, i, i + 1);
    }
    reserve();
}

void PrefixTree::clear() {
    while (!tails_.empty()) remove_seq((int)tails_.size() - 1);
}

std::vector<ca_chunk_info> PrefixTree::get_chunks() const {
    // Pre-order with an explicit stack; children are pushed first to last and therefore visited
    // last to first, a parent always before its children.  Empty reserved tails are listed too:
    // they receive the next appended token without a change of the work list.
    std::vector<ca_chunk_info> infos;
    std::vector<std::pair<int, const Chunk*>> stack;
    infos.reserve(1024);
    stack.reserve(1024);
    stack.emplace_back(0, root_.get());
    while (!stack.empty()) {
        const int seq_begin = stack.back().first;
        const Chunk* chunk = stack.back().second;
        stack.pop_back();
        int start = seq_begin;
        for (const Chunk* child : chunk->children) {
            stack.emplace_back(start, child);
            start += child->n_seqs;
        }
        if (chunk == root_.get()) continue;
        infos.push_back(ca_chunk_info{chunk->id, chunk->n_tokens(), seq_begin, seq_begin + chunk->n_seqs});
    }
    return infos;
}

}  // namespace ca_host
