"""In-repo KV block store: pinned host DRAM shared by every rank of a node.

``KvStore`` (C++, csrc/store/kvstore.cpp) is the shared-memory index + arena; ``PinnedKVStore``
binds one rank's paged cache to it and moves blocks with the transfer kernels.
"""
from .store import PinnedKVStore, block_keys, store_format, store_page_layout, store_salt  # noqa: F401
