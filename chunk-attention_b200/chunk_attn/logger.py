"""The package logger, `chunk_attn.logger.logger` as in the reference (src/chunk_attn/logger.py:4-12): name
"ChunkAttn", messages to stdout with time, level and process:thread.  Level from CHUNK_ATTN_LOG (default INFO)."""
import logging
import os
import sys

logger = logging.getLogger("ChunkAttn")
logger.setLevel(getattr(logging, os.environ.get("CHUNK_ATTN_LOG", "INFO").upper(), logging.INFO))
if not logger.handlers:
    _handler = logging.StreamHandler(sys.stdout)
    _handler.setFormatter(logging.Formatter(
        "[%(asctime)s] [%(name)s] [%(levelname)s] [%(process)d:%(thread)d] %(message)s"))
    logger.addHandler(_handler)
    logger.propagate = False
