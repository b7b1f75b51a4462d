"""Rank-aware logging helpers (reference ``utils/log_utils.py:1-23``)."""
from __future__ import annotations

import logging
import os

import torch


def get_logger(name: str = "odysseus_b200") -> logging.Logger:
    logger = logging.getLogger(name)
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(message)s"))
        logger.addHandler(h)
        logger.setLevel(os.environ.get("ODY_LOGLEVEL", "INFO"))
        logger.propagate = False
    return logger


def rank_log(rank: int, logger: logging.Logger, msg: str) -> None:
    """Log on rank 0 only."""
    if rank == 0:
        logger.info(msg)


def verify_min_gpu_count(min_gpus: int = 2) -> bool:
    return torch.cuda.is_available() and torch.cuda.device_count() >= min_gpus
