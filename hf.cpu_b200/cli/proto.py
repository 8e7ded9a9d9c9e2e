"""The stdin/stdout event protocol (docs/PROTOCOL.md; src/proto.c).

Responses are event lines ``@name key=value ...``; a value is quoted when it is empty or contains a
character <= space, a quote, a backslash, ``=`` or DEL, with ``\\"``, ``\\\\``, ``\\n``, ``\\r``, ``\\t`` and
``\\xHH`` escapes inside the quotes (src/proto.c:111-138).  Requests are records on stdin separated by a
byte; a record larger than the limit is skipped and reported, and the stream stays in sync
(src/proto.c:51-99).
"""
from __future__ import annotations

import os
from typing import BinaryIO, Iterator, Optional, Tuple


def quote(v: str) -> str:
    need = v == "" or any(ord(c) <= 0x20 or c in '"\\=' or ord(c) == 0x7F for c in v)
    if not need:
        return v
    out = ['"']
    for c in v:
        if c in '"\\':
            out.append("\\" + c)
        elif c == "\n":
            out.append("\\n")
        elif c == "\r":
            out.append("\\r")
        elif c == "\t":
            out.append("\\t")
        elif ord(c) < 0x20 or ord(c) == 0x7F:
            out.append(f"\\x{ord(c):02x}")
        else:
            out.append(c)
    out.append('"')
    return "".join(out)


class EventWriter:
    def __init__(self, f: BinaryIO):
        self.f, self.err = f, False

    def _put(self, data: bytes) -> None:
        if self.err:
            return
        try:
            self.f.write(data)
        except (BrokenPipeError, OSError):
            self.err = True

    def event(self, name: str, /, **pairs) -> None:
        parts = ["@" + name] + [f"{k}={quote('' if v is None else str(v))}" for k, v in pairs.items()]
        self._put((" ".join(parts) + "\n").encode("utf-8", "surrogateescape"))
        self.flush()

    def payload(self, name: str, data: bytes, **pairs) -> None:
        parts = [f"@{name} len={len(data)}"] + [f"{k}={quote(str(v))}" for k, v in pairs.items()]
        self._put((" ".join(parts) + "\n").encode() + data + b"\n")
        self.flush()

    def raw_byte(self, b: int) -> None:
        self._put(bytes([b]))

    def flush(self) -> None:
        if self.err:
            return
        try:
            self.f.flush()
        except (BrokenPipeError, OSError):
            self.err = True


class RecordReader:
    """Yields ``(status, record)``: status None for a record, ``"ERANGE"`` for one that was too large
    (skipped up to its separator)."""

    def __init__(self, fd: int = 0):
        self.fd, self.buf, self.eof = fd, bytearray(), False

    def _fill(self) -> bool:
        if self.eof:
            return False
        chunk = os.read(self.fd, 1 << 16)
        if not chunk:
            self.eof = True
            return False
        self.buf += chunk
        return True

    def next(self, sep: int, max_record: int) -> Optional[Tuple[Optional[str], bytes]]:
        skipping = False
        scanned = 0
        while True:
            i = self.buf.find(bytes([sep]), scanned)
            if i >= 0:
                rec = bytes(self.buf[:i])
                del self.buf[:i + 1]
                if skipping or len(rec) > max_record:
                    return ("ERANGE", b"")
                return (None, rec)
            scanned = len(self.buf)
            if len(self.buf) > max_record:
                skipping = True
                del self.buf[:]
                scanned = 0
            if not self._fill():
                if skipping:
                    return ("ERANGE", b"")
                if self.buf:
                    rec = bytes(self.buf)
                    del self.buf[:]
                    return (None, rec)
                return None
