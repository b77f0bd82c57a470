"""Continuous-batching loop around a model and its per-layer KV caches.

Surface and iteration order of the reference's ModelHost (src/chunk_attn/models/model_host.py:13-134):
every iteration (1) retires finished sequences from every cache, (2) prefills the requests that
arrived, inserting each at the row its prefill returned, (3) runs one decode step over everything
that is running.  `running_seqs` is therefore always in the caches' DFS row order, which is the
order `Attention.forward` expects its query rows in.

Unlike the reference, an exception on the worker thread does not leave callers blocked: it is
handed to every sequence in flight and to every later `predict`.
"""
import queue
import threading

import torch

from ..logger import logger
from .sequence import Sequence


class ModelHost:
    def __init__(self, model_obj, kv_caches, max_batch_size=32):
        self.model_obj = model_obj
        self.kv_caches = kv_caches
        self.running_seqs = []
        self.max_batch_size = max_batch_size
        self.peak_batch_size = 0
        self.stopped = True
        self.cycle_time = 1.0
        self.failure = None
        self.n_decode_steps = 0
        self.batch_queue = queue.Queue(maxsize=2 * max_batch_size)
        self.thread = None

    # ---- client side ---------------------------------------------------------------------------
    def predict_async(self, prompt_tokens, max_tokens):
        if self.failure is not None:
            raise RuntimeError("model host failed: %r" % (self.failure,))
        if self.stopped:
            raise RuntimeError("model host is stopped, can't predict anymore")
        if len(prompt_tokens) == 0:
            raise ValueError("empty prompt")
        seq = Sequence(prompt_tokens=prompt_tokens, max_tokens=max_tokens)
        self.batch_queue.put(seq)
        return seq

    def predict(self, prompt_tokens, max_tokens):
        return self.predict_async(prompt_tokens, max_tokens).get_result()

    def start(self):
        if not self.stopped:
            raise RuntimeError("model host is already started")
        self.stopped = False
        self.thread = threading.Thread(target=self.run_iterations, name="chunk-attn-model-host", daemon=True)
        self.thread.start()

    def stop(self):
        self.stopped = True
        if self.thread is not None:
            self.thread.join()
            self.thread = None

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.stop()

    # ---- worker side ---------------------------------------------------------------------------
    def get_new_requests(self):
        new_seqs = []
        if len(self.running_seqs) == 0:  # idle: block until something arrives (or a cycle passes)
            try:
                new_seqs.append(self.batch_queue.get(block=True, timeout=self.cycle_time))
            except queue.Empty:
                pass
        while len(new_seqs) + len(self.running_seqs) < self.max_batch_size:
            try:
                new_seqs.append(self.batch_queue.get(block=False))
            except queue.Empty:
                break
        return new_seqs

    def retire_finished(self):
        """Drop finished sequences from the batch and from every layer's cache (rows shift down as the
        reference's index arithmetic assumes, model_host.py:88-102)."""
        kept = []
        n_removed = 0
        for idx, seq in enumerate(self.running_seqs):
            if seq.finished():
                for kv_cache in self.kv_caches:
                    kv_cache.remove_seq(idx - n_removed)
                n_removed += 1
                logger.debug("finished the seq %s", seq.id)
                seq.set_result_ready()
            else:
                kept.append(seq)
        self.running_seqs = kept
        return n_removed

    def step(self):
        """One iteration of the serving loop; returns the number of sequences that were decoded."""
        self.retire_finished()
        arrived = self.get_new_requests()
        if arrived:
            logger.debug("prefill of %d new seqs, %d running", len(arrived), len(self.running_seqs))
            new_tokens = self.model_obj(arrived, self.kv_caches, prefill=True)
            for seq, tok in zip(arrived, new_tokens):
                seq.append(tok)
            for seq in arrived:  # same order as the caches inserted them: rows stay aligned
                self.running_seqs.insert(seq.index, seq)
        self.peak_batch_size = max(self.peak_batch_size, len(self.running_seqs))
        # a one-token request is complete after its prefill; it must not be decoded
        live = [s for s in self.running_seqs if not s.finished()]
        if len(live) != len(self.running_seqs):
            self.retire_finished()
        if self.running_seqs:
            new_tokens = self.model_obj(self.running_seqs, self.kv_caches, prefill=False)
            for seq, tok in zip(self.running_seqs, new_tokens):
                seq.append(tok)
            self.n_decode_steps += 1
        return len(self.running_seqs)

    @torch.inference_mode()
    def run_iterations(self):
        try:
            while not self.stopped:
                self.step()
            # a stop request lets nothing hang: whatever is still running leaves the caches (last row
            # first, so the remaining rows keep their indices) and is reported as cancelled
            for idx in reversed(range(len(self.running_seqs))):
                for kv_cache in self.kv_caches:
                    kv_cache.remove_seq(idx)
            self._fail_all(RuntimeError("model host stopped before the sequence finished"), record=False)
        except BaseException as e:  # noqa: BLE001 - handed to the callers, not swallowed
            self._fail_all(e, record=True)

    def _fail_all(self, error, record):
        if record:
            logger.error("model host failed: %r", error)
            self.failure = error
            self.stopped = True
        for seq in self.running_seqs:
            seq.set_error(error)
        self.running_seqs = []
        while True:
            try:
                self.batch_queue.get(block=False).set_error(error)
            except queue.Empty:
                break
