"""Logging with a per-rank prefix and an environment-controlled level
(reference: mindspeed/log_config.py:10-70; env ``MIND_SPEED_LOG_LEVEL``)."""
from __future__ import annotations

import logging
import logging.config
import os

import torch.distributed as dist

_LEVEL_ENV = "MIND_SPEED_LOG_LEVEL"
_warned = set()


def _rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else int(os.environ.get("RANK", 0))


def set_log_config():
    level = os.environ.get(_LEVEL_ENV, "INFO").upper()
    if level not in ("DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"):
        level = "INFO"
    logging.config.dictConfig({
        "version": 1, "disable_existing_loggers": False,
        "formatters": {"rank": {"format": f"[Rank {_rank()} | Local Rank {os.environ.get('LOCAL_RANK', 0)}] "
                                          "%(asctime)s %(levelname)s %(name)s: %(message)s"}},
        "handlers": {"console": {"class": "logging.StreamHandler", "formatter": "rank", "level": level}},
        "loggers": {"mindspeed_b200": {"handlers": ["console"], "level": level, "propagate": False}},
    })


def get_logger(name="mindspeed_b200"):
    return logging.getLogger(name)


def print_rank_0(msg):
    if _rank() == 0:
        print(msg, flush=True)


def print_rank_last(msg):
    last = dist.get_world_size() - 1 if dist.is_available() and dist.is_initialized() else 0
    if _rank() == last:
        print(msg, flush=True)


def log_rank_0(logger, level, msg):
    if _rank() == 0:
        logger.log(level, msg)


def log_warning_once(logger, msg):
    if msg not in _warned:
        _warned.add(msg)
        logger.warning(msg)
