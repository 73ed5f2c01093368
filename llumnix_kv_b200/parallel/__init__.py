"""Multi-GPU building blocks that sit beside the point-to-point transfer.

The KV transfer itself is a push from one GPU into another's memory (``csrc/transport/nvlink_channel.cpp``
and ``csrc/kernels/kvt_p2d_attn.cu``); this package holds what involves a group of GPUs:

``nvls``  ``MulticastKVCache``: paged caches of a decode TP group in memory bound to an NVLink multicast
          object, and the relay that replicates pages every rank holds identically (MLA latent, indexer
          cache, replicated KV heads) with ``multimem.st`` through NVSwitch.
"""
