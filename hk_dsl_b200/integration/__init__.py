"""Engine routes of this build: switches, the patch/op contract, the vLLM attention backend
and the in-place attention stand-ins (the part of hk-dsl's `hk.integration` that serves the
paged KV path)."""
