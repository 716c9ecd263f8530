"""Host side of the paged KV kernels (mirrors the decode half of hk-dsl's `hk.ops.paged`)."""
