"""Minimal JSON-lines training logger with an elapsed-time field (API of
torchsso/utils/logger.py:8-45; application-level helper, not on the curvature path)."""
import json
import os
import shutil
import tempfile
import time


class Logger(object):

    def __init__(self, out, logname):
        self.out = out
        self.logname = logname
        self._log = []
        self._start_at = None
        os.makedirs(out, exist_ok=True)

    def start(self, start_at=None):
        self._start_at = time.time() if start_at is None else start_at

    @property
    def elapsed_time(self):
        if self._start_at is None:
            raise RuntimeError('training has not been started yet')
        return time.time() - self._start_at

    def write(self, log):
        self._log.append(log)
        fd, path = tempfile.mkstemp(prefix=self.logname, dir=self.out)
        with os.fdopen(fd, 'w') as f:
            json.dump(self._log, f, indent=4)
        shutil.move(path, os.path.join(self.out, self.logname))
