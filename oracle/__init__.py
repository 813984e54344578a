"""CPU restatement of the reference's paged KV-cache path (CoLearn-Dev/deserve).

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this; it is
the checker used by tests/, by __graft_entry__.smoke() and by bench.py's CPU
baseline / reference arm. It restates, in plain numpy / CPU torch and
parameterised in (n_kv_heads, head_dim, page_size, dtype), what the reference
does with torch on a device:

  paged_alloc.py  page pool bitmap allocator, page-table slots, per-sequence
                  growth, the two-region virtual pool and the buddy chunk pool
  descriptors.py  TaskData stepping and the ragged-batch descriptor build
  kv_math.py      append-scatter, K/V gather through the page table, rotary
                  embedding, dense fp32 attention (decode and causal prefill)
  swap_ops.py     region swap, per-task offload / reload chunk layout

Parity pin: the integer paths (allocator order, page tables, descriptors,
region state machine, buddy pool, offload chunk layout) and the dense fp32
attention + rotary math are pinned against outputs of the reference's own
classes run on CPU (tests/golden/make_golden.py imports them from the
reference tree and writes tests/golden/*.json|npz). The paged append, the
paged attention kernels, the in-place rotary embedding and RMSNorm exist in
the reference only as calls into the third-party flashinfer package (version
not pinned, no tests in the reference): the oracle states their call
semantics (index rule + the dense attention math applied to K/V gathered
through the page table) and is pinned at that boundary against results
recorded from flashinfer 0.6.11 itself on a B200
(tests/golden/make_flashinfer_golden.py -> tests/golden/flashinfer_golden.*).
"""
