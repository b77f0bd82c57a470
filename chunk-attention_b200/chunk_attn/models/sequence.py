"""One request in flight (surface of the reference's src/chunk_attn/models/sequence.py:6-36)."""
import itertools
import threading

_ids = itertools.count()


class Sequence:
    """Prompt + generated tokens.  `index` is the row the sequence occupies in the KV caches' DFS
    order (set by the model's prefill); `get_result()` blocks until the host marks it finished or
    failed."""

    def __init__(self, prompt_tokens, max_tokens=2048):
        self.id = "seq-%d" % next(_ids)
        self.prompt_tokens = list(prompt_tokens)
        self.max_tokens = max_tokens
        self.tokens = list(self.prompt_tokens)
        self.index = None
        self.error = None
        self.result_ready = threading.Event()

    def get_result(self, timeout=None):
        if not self.result_ready.wait(timeout):
            raise TimeoutError("sequence %s is not finished" % self.id)
        if self.error is not None:
            raise self.error
        return self.tokens

    def set_result_ready(self):
        self.result_ready.set()

    def set_error(self, error):
        self.error = error
        self.result_ready.set()

    def append(self, token):
        self.tokens.append(token)

    def finished(self):
        return len(self.tokens) >= self.max_tokens + len(self.prompt_tokens)

    def __len__(self):
        return len(self.tokens)

    def __getitem__(self, index):
        return self.tokens[index]
