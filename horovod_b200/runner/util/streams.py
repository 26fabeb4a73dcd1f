"""A one-slot pipe between two threads: the writer blocks until the reader has
taken the previous piece; works with str and bytes.
Parity: horovod/runner/util/streams.py (Pipe)."""
import threading


class Pipe:
    def __init__(self):
        self._cv = threading.Condition()
        self._piece = None   # what was written and not fully read yet
        self._pos = 0
        self._closed = False

    def write(self, buf):
        with self._cv:
            self._cv.wait_for(lambda: self._piece is None or self._closed)
            if self._closed:
                raise RuntimeError("Pipe is closed")
            self._piece, self._pos = buf, 0
            self._cv.notify_all()

    def read(self, length=-1):
        """Up to ``length`` items of the current piece (all of it when length
        is not positive); blocks until something was written; None once the
        pipe is closed and drained."""
        with self._cv:
            self._cv.wait_for(lambda: self._piece is not None or self._closed)
            if self._piece is None:
                return None
            left = len(self._piece) - self._pos
            if 0 < length < left:
                out = self._piece[self._pos:self._pos + length]
                self._pos += length
            else:
                out = self._piece[self._pos:]
                self._piece = None
            self._cv.notify_all()
            return out

    def flush(self):
        pass

    def close(self):
        with self._cv:
            self._closed = True
            self._cv.notify_all()
