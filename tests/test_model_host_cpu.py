"""ModelHost's batching and row bookkeeping on the CPU: a stand-in model that keeps one real
PrefixTree per layer (the compiled host tree runs without a GPU) and emits a deterministic next
token, so every request's output is known in advance and the batch order can be compared with the
trees' row order at every step."""
import random
import threading
import time

import pytest

from chunk_attn import PrefixTree
from chunk_attn.models.model_host import ModelHost
from chunk_attn.models.sequence import Sequence


def next_token(tokens):
    return 1000 + (sum(tokens) * 31 + len(tokens) * 7) % 977


def rollout(prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(next_token(toks))
    return toks


def tree_rows(tree):
    """Token list of every sequence in the tree's row (DFS) order."""
    rows = []

    def walk(node, prefix):
        here = prefix + list(node.tokens)
        if not node.children:
            rows.append(here)
        for c in node.children:
            walk(c, here)

    for c in tree.get_trie().children:
        walk(c, [])
    return rows


class TreeCache:
    def __init__(self):
        self.tree = PrefixTree(chunk_size=4, max_chunks=4096)

    def remove_seq(self, i):
        self.tree.remove_seq(i)


class TreeModel:
    """Makes the calls the decoder makes, on every layer's tree, and checks the batch order."""

    def __init__(self, fail_at_decode=None):
        self.decodes = 0
        self.prefills = 0
        self.fail_at_decode = fail_at_decode
        self.max_batch = 0

    def __call__(self, seqs, kv_caches, prefill):
        if prefill:
            self.prefills += 1
            for s in seqs:
                idx = {c.tree.add_seq(s.tokens) for c in kv_caches}
                assert len(idx) == 1  # every layer agrees on the row
                s.index = idx.pop()
        else:
            self.decodes += 1
            if self.fail_at_decode is not None and self.decodes >= self.fail_at_decode:
                raise RuntimeError("injected model failure")
            self.max_batch = max(self.max_batch, len(seqs))
            for c in kv_caches:
                # rows of the tree (without the token being fed now) == the batch, in order
                assert tree_rows(c.tree) == [s.tokens[:-1] for s in seqs]
                c.tree.append_token([s[-1] for s in seqs])
                c.tree.reserve()
        return [next_token(s.tokens) for s in seqs]


def make_host(max_batch_size=8, layers=2, **kw):
    caches = [TreeCache() for _ in range(layers)]
    host = ModelHost(TreeModel(**kw), caches, max_batch_size=max_batch_size)
    host.cycle_time = 0.05
    return host, caches


def test_sequence_surface():
    s = Sequence([1, 2, 3], max_tokens=2)
    assert len(s) == 3 and s[-1] == 3 and s.index is None and not s.finished()
    s.append(4)
    s.append(5)
    assert s.finished() and s.tokens == [1, 2, 3, 4, 5]
    with pytest.raises(TimeoutError):
        s.get_result(timeout=0.01)
    s.set_result_ready()
    assert s.get_result() == [1, 2, 3, 4, 5]
    s2 = Sequence([1])
    s2.set_error(ValueError("x"))
    with pytest.raises(ValueError):
        s2.get_result()


def test_single_request_matches_rollout():
    host, caches = make_host()
    with host:
        assert host.predict([5, 6, 7], 9) == rollout([5, 6, 7], 9)
    assert all(tree_rows(c.tree) == [] for c in caches)


def test_predict_refused_when_stopped_and_double_start():
    host, _ = make_host()
    with pytest.raises(RuntimeError, match="stopped"):
        host.predict_async([1], 1)
    host.start()
    with pytest.raises(RuntimeError, match="already started"):
        host.start()
    host.stop()


def test_shared_prefix_requests_in_waves():
    """Requests with shared prefixes arriving while others decode: insertion rows, removals on finish
    and the batch limit all have to keep the batch aligned with the trees (checked inside the model)."""
    rnd = random.Random(4)
    host, caches = make_host(max_batch_size=6)
    system = [rnd.randrange(100) for _ in range(11)]
    prompts = []
    for i in range(20):
        own = [rnd.randrange(100, 200) for _ in range(rnd.randrange(1, 9))]
        prompts.append((system + own) if i % 3 else own)
    lens = [rnd.randrange(1, 14) for _ in prompts]
    with host:
        pending = []
        for i, (p, n) in enumerate(zip(prompts, lens)):
            pending.append(host.predict_async(p, n))
            if i % 5 == 4:
                pending[i - 2].get_result(timeout=20)  # let some finish before the next wave
        results = [s.get_result(timeout=20) for s in pending]
    for p, n, r in zip(prompts, lens, results):
        assert r == rollout(p, n)
    assert host.peak_batch_size <= 6 and host.model_obj.max_batch <= 6
    assert host.model_obj.max_batch >= 2  # requests really were batched
    assert all(tree_rows(c.tree) == [] for c in caches)


def test_concurrent_clients():
    host, caches = make_host(max_batch_size=4)
    out = {}

    def client(i):
        out[i] = host.predict([i, i + 1, 50, 51, 52], 6 + i % 3)

    with host:
        threads = [threading.Thread(target=client, args=(i,)) for i in range(10)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(30)
    assert all(out[i] == rollout([i, i + 1, 50, 51, 52], 6 + i % 3) for i in range(10))


def test_one_token_request_is_not_decoded():
    host, _ = make_host()
    with host:
        assert host.predict([9, 9, 9], 1) == rollout([9, 9, 9], 1)
    assert host.model_obj.decodes == 0


def test_model_failure_reaches_every_caller():
    host, _ = make_host(fail_at_decode=3)
    host.start()
    a = host.predict_async([1, 2, 3], 50)
    b = host.predict_async([1, 2, 4], 50)
    for s in (a, b):
        with pytest.raises(RuntimeError, match="injected model failure"):
            s.get_result(timeout=20)
    host.thread.join(10)
    with pytest.raises(RuntimeError, match="model host failed"):
        host.predict_async([1], 1)
    host.stop()


def test_stop_cancels_running_sequences_and_cleans_the_caches():
    host, caches = make_host()
    host.start()
    s = host.predict_async([1, 2, 3], 10 ** 9)
    deadline = time.monotonic() + 20
    while host.n_decode_steps < 3 and host.failure is None:
        assert time.monotonic() < deadline, "the worker made no progress"
        time.sleep(0.001)
    host.stop()
    with pytest.raises(RuntimeError, match="stopped before"):
        s.get_result(timeout=5)
    assert all(tree_rows(c.tree) == [] for c in caches)


def test_step_api_without_a_thread():
    host, caches = make_host()
    host.stopped = False
    a = host.predict_async([1, 2, 3, 4, 5, 6], 2)
    b = host.predict_async([1, 2, 3, 4, 9], 3)
    assert host.step() == 2  # prefill both + one decode
    assert [s.tokens[:-1] for s in host.running_seqs] == tree_rows(caches[0].tree)
    assert host.step() == 1  # a finished (2 tokens) and retired; b decoded
    assert a.result_ready.is_set() and a.tokens == rollout([1, 2, 3, 4, 5, 6], 2)
    host.step()
    assert b.result_ready.is_set() and b.tokens == rollout([1, 2, 3, 4, 9], 3)


def test_helper_modules_of_the_reference_package_exist():
    import chunk_attn.nvtx as nvtx
    from chunk_attn.logger import logger
    nvtx.range_push("x")
    nvtx.range_pop()
    assert logger.name == "ChunkAttn"
