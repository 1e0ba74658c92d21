"""Stand-in for the `xxhash` package, which the reference's block manager imports
(nanovllm/engine/block_manager.py:3) and this environment does not ship.  Only the
xxh64 surface the reference uses is provided: update() and intdigest().  The hash
function differs from real xxHash; the reference only needs a stable 64-bit content
hash for prefix caching, so behaviour is unchanged."""
import hashlib


class xxh64:
    def __init__(self, data=b""):
        self._h = hashlib.blake2b(digest_size=8)
        if data:
            self._h.update(data)

    def update(self, data):
        self._h.update(bytes(data))

    def intdigest(self):
        return int.from_bytes(self._h.digest(), "little")

    def digest(self):
        return self._h.digest()

    def hexdigest(self):
        return self._h.hexdigest()
