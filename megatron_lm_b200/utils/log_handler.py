"""Logging set-up of the training programs: records go to stdout, records of chatty third-party loggers are dropped,
and ``--logging-level`` (or the ``MEGATRON_LOGGING_LEVEL`` variable) sets the level
(reference: megatron/training/log_handler.py:9 CustomHandler, megatron/training/initialize.py setup_logging)."""
import logging
import os
import sys

QUIET_LOGGERS = ["torch.distributed"]


class StdoutHandler(logging.StreamHandler):
    def __init__(self, quiet=None):
        super().__init__(stream=sys.stdout)
        self.quiet = list(QUIET_LOGGERS if quiet is None else quiet)

    def filter(self, record: logging.LogRecord) -> bool:
        return not any(record.name.startswith(q) for q in self.quiet)


CustomHandler = StdoutHandler        # the reference's name


def setup_logging(level=None) -> int:
    """Installs the handler on the root logger once; precedence of the level: argument, environment, INFO."""
    if level is None:
        env = os.environ.get("MEGATRON_LOGGING_LEVEL")
        level = int(env) if env else logging.INFO
    root = logging.getLogger()
    if not any(isinstance(h, StdoutHandler) for h in root.handlers):
        root.addHandler(StdoutHandler())
    root.setLevel(level)
    return level
