"""KV swap on the GPU against the oracle: region swap, pack / unpack, and the
per-task offload / reload into different page ids — all bit-exact."""
import numpy as np
import pytest
import torch

import deserve_b200 as dk
from deserve_b200 import _lib
from oracle import swap_ops
from oracle.paged_alloc import OracleVirtualPool

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _fill(pool, seed):
    g = torch.Generator().manual_seed(seed)
    cpu = torch.randn(pool.pages.shape, generator=g).to(pool.main_dtype)
    pool.pages.copy_(cpu)
    return cpu


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    assert _lib.read_device_status() == 0, "a kernel self-check fired"


@pytest.mark.parametrize("dtype,layers", [(torch.bfloat16, 5), (torch.float16, 1), (torch.float32, 8)])
@pytest.mark.parametrize("whole", [True, False])
def test_region_swap_bit_exact(dtype, layers, whole):
    """whole: every byte of the region travels, the reference's statement of the swap
    (VirtualPagePool.swap(), virtual.py:97-113). Otherwise swap2 moves only the head of each
    region up to its highest page in use: 2 of 4 pages leave, 3 of 4 arrive, the free tails stay
    where they are on both sides."""
    main, swap, ps, hkv, d = 6, 4, 16, 2, 64
    pool = dk.VirtualPagePool(layers, main, swap, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    ref = _fill(pool, 1)
    size = pool.calc_swap_size()
    prev_mb = dk.CopiedPinnedMemory(size, swap, DEV, dtype)
    next_mb = dk.CopiedPinnedMemory(size, swap, DEV, dtype)
    incoming = torch.randn(size, generator=torch.Generator().manual_seed(2)).to(dtype)
    next_mb.memory.copy_(incoming)
    prev_mb.memory.zero_()
    want_out = torch.zeros(size, dtype=dtype)
    lo, hi = pool.slices[1 - pool.on]
    if whole:
        swap_ops.region_swap(ref, lo, hi, want_out, incoming)
        pool.swap(next_mb, prev_mb)
    else:
        pool._swap_bitmap[:2] = False                 # the region going out has pages 0 and 1 in use
        next_mb.bitmap[[0, 2]] = False                # the one coming in pages 0 and 2: its head is 3 pages long
        shape = (layers, swap, *ref.shape[2:])
        want_out.view(shape)[:, :2] = ref[:, lo : lo + 2]
        ref[:, lo : lo + 3] = incoming.view(shape)[:, :3]
        pool.swap2(next_mb, prev_mb)
        assert pool.last_swap_pages == (2, 3)
    pool.stream.synchronize()
    pool.stream2.synchronize()
    assert torch.equal(prev_mb.memory.view(torch.uint8), want_out.view(torch.uint8))
    assert torch.equal(pool.pages.cpu().view(torch.uint8), ref.view(torch.uint8))


def test_region_swap_moves_only_the_token_rows_in_use():
    """The step builder tells the pool how many token rows of its region pages hold data (note_rows);
    swap2 then moves only those rows of each half page (K rows, V rows), both ways, and the row counts
    travel with the host image. Everything else stays as it was on both sides."""
    layers, main, swap, ps, hkv, d, dtype = 3, 6, 4, 16, 2, 64, torch.bfloat16
    pool = dk.VirtualPagePool(layers, main, swap, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    ref = _fill(pool, 3)
    size = pool.calc_swap_size()
    prev_mb = dk.CopiedPinnedMemory(size, swap, DEV, dtype)
    next_mb = dk.CopiedPinnedMemory(size, swap, DEV, dtype)
    incoming = torch.randn(size, generator=torch.Generator().manual_seed(4)).to(dtype)
    next_mb.memory.copy_(incoming)
    prev_mb.memory.zero_()
    lo, hi = pool.slices[1 - pool.on]
    pool._swap_bitmap[:2] = False                 # going out: pages 0 and 1 in use, holding 5 and 3 tokens
    pool.note_rows(np.array([lo, lo + 1]), np.array([lo, lo + 1]), np.array([5, 3]))
    next_mb.bitmap[[0, 2]] = False                # coming in: pages 0 and 2 in use, 7 and 2 tokens; page 1 is free
    next_mb.rows = np.array([7, 16, 2, 16], dtype=np.int32)
    pool.swap2(next_mb, prev_mb)
    assert pool.last_swap_pages == (2, 3) and pool.last_swap_rows == (5, 7)
    assert prev_mb.rows.tolist() == [5, 3, 16, 16]
    rel = lo - main
    assert pool.rows_used[rel : rel + swap].tolist() == [7, 16, 2, 16]
    pool.stream.synchronize()
    pool.stream2.synchronize()
    # pages are [K|V][token][head][dim]: rows = tokens of each half
    shape = (layers, swap, 2, ps, hkv, d)
    want_out = torch.zeros(shape, dtype=dtype)
    want_out[:, :2, :, :5] = ref[:, lo : lo + 2, :, :5]
    assert torch.equal(prev_mb.memory.view(torch.uint8), want_out.view(-1).view(torch.uint8))
    ref[:, lo : lo + 3, :, :7] = incoming.view(shape)[:, :3, :, :7]
    assert torch.equal(pool.pages.cpu().view(torch.uint8), ref.view(torch.uint8))
    # a page that is freed is a whole page again for whoever gets it next
    pool.free(np.array([lo]))
    assert pool.rows_used[rel] == ps


def test_region_state_machine_with_data_follows_a_microbatch():
    """Two microbatches share one pool: each one's swap-region pages leave to its
    pinned buffer while the other computes and come back intact (rounds = 3, so
    a microbatch alternates regions and its page ids are shifted by adjust)."""
    L, main, swap, ps, hkv, d = 2, 4, 3, 8, 2, 64
    rounds = 3
    pool = dk.VirtualPagePool(L, main, swap, ps, DEV, torch.bfloat16, n_kv_heads=hkv, head_dim=d)
    pool.pages.zero_()
    pta = dk.PageTableAllocator(16, 1024, ps, DEV)
    pinned = [dk.CopiedPinnedMemory(pool.calc_swap_size(), swap, DEV, torch.bfloat16) for _ in range(rounds)]
    for p in pinned:
        p.memory.zero_()
    caches = [None] * rounds
    stamp = {}
    for step in range(4 * rounds):
        mb = step % rounds
        pool.stream.synchronize()
        pool.stream2.synchronize()
        pool.switch()
        if caches[mb] is not None:
            offset = pool.num_pages_swap if pool.on == 1 else -pool.num_pages_swap
            caches[mb].adjust(offset)
            ids = caches[mb].page_table.retrieve().tolist()
            for j, pid in enumerate(ids):  # pages are where the table says, with this microbatch's stamp
                assert pool.pages[:, pid].float().unique().tolist() == [stamp[(mb, j)]], (step, mb, j, pid)
        else:
            caches[mb] = dk.VirtualPagedKVCache.empty(pta, pool)
            caches[mb].extend([6, 3, 2][mb] * ps)  # mb0: 4 main + 2 region pages; mb1, mb2: region pages only
            for j, pid in enumerate(caches[mb].page_table.retrieve().tolist()):
                stamp[(mb, j)] = float(10 * (mb + 1) + j)
                pool.pages[:, pid] = stamp[(mb, j)]
        pool.swap2(pinned[(mb + 1) % rounds], pinned[(mb - 1 + rounds) % rounds])
    pool.stream.synchronize()
    pool.stream2.synchronize()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_pack_unpack_roundtrip_bit_exact(dtype):
    L, P, ps, hkv, d = 4, 40, 16, 2, 64
    pool = dk.GpuPagePool(L, P, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    ref = _fill(pool, 3)
    rng = np.random.default_rng(0)
    counts = [5, 1, 9]
    perm = rng.permutation(P)
    id_lists = np.split(perm[: sum(counts)], np.cumsum(counts)[:-1])
    ids = torch.tensor(np.concatenate(id_lists), dtype=torch.int32, device=DEV)
    indptr = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    for l0, l1 in [(0, L), (1, 3)]:
        w = l1 - l0
        packed = torch.zeros(sum(counts) * w, *pool.pages.shape[2:], dtype=dtype, device=DEV)
        _lib.check(_lib.lib.dsv_pack_pages(pool.pages.data_ptr(), pool.layer_stride_bytes, pool.page_bytes, P,
                                           ids.data_ptr(), indptr.data_ptr(), len(counts), sum(counts), l0, l1,
                                           packed.data_ptr(), _lib.current_stream_ptr(DEV)))
        want = torch.cat([swap_ops.offload_rows(ref[l0:l1], x) for x in id_lists])
        assert torch.equal(packed.cpu().view(torch.uint8), want.view(torch.uint8))
        # scatter into a different page assignment
        perm2 = rng.permutation(P)
        id_lists2 = np.split(perm2[: sum(counts)], np.cumsum(counts)[:-1])
        ids2 = torch.tensor(np.concatenate(id_lists2), dtype=torch.int32, device=DEV)
        before = pool.pages.cpu()
        _lib.check(_lib.lib.dsv_unpack_pages(packed.data_ptr(), pool.pages.data_ptr(), pool.layer_stride_bytes,
                                             pool.page_bytes, P, ids2.data_ptr(), indptr.data_ptr(), len(counts),
                                             sum(counts), l0, l1, _lib.current_stream_ptr(DEV)))
        at = 0
        for x, n in zip(id_lists2, counts):
            swap_ops.reload_rows(before[l0:l1], x, want[at : at + n * w])
            at += n * w
        assert torch.equal(pool.pages.cpu().view(torch.uint8), before.view(torch.uint8))
        ref = before


@pytest.mark.parametrize("staging_kib", [None, 160])
def test_offload_reload_into_new_pages_bit_exact(staging_kib):
    """KVCacheManager: offload several tasks to pinned chunks, free and reuse
    their pages, reload into freshly allocated ids. The small staging size forces
    several layer windows through the double buffer."""
    L, main, swap, ps, hkv, d = 6, 40, 4, 16, 2, 64
    dtype = torch.bfloat16
    pool = dk.VirtualPagePool(L, main, swap, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    ref = _fill(pool, 4)
    o_pool = OracleVirtualPool(main, swap, ps)
    pta = dk.PageTableAllocator(16, 4096, ps, DEV)
    chunks = dk.CpuChunkPool(L, 6, ps, dtype, n_kv_heads=hkv, head_dim=d)
    mgr = dk.KVCacheManager(pool, chunks, pta, staging_bytes=None if staging_kib is None else staging_kib << 10)
    caches = []
    for tokens in (5 * ps, 1, 9 * ps - 3):
        c = dk.VirtualPagedKVCache.empty(pta, pool)
        c.extend(tokens)
        caches.append(c)
    id_lists = [c.page_table.retrieve().numpy().copy() for c in caches]
    handles = mgr.offload_many(caches)
    for c in caches:
        c.free()
    mgr.synchronize()
    mgr.dma_stream.synchronize()
    rows = [swap_ops.offload_rows(ref, ids) for ids in id_lists]
    for h, want, ids in zip(handles, rows, id_lists):
        got = h.retrieve()[: len(ids) * L]
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    # overwrite the freed pages, then reload into whatever ids the pool hands out
    pool.pages[:, torch.as_tensor(np.concatenate(id_lists), dtype=torch.long, device=DEV)] = -7.0
    ref = pool.pages.cpu()
    filler = dk.VirtualPagedKVCache.empty(pta, pool)
    filler.extend(3 * ps)
    new_caches = mgr.reload_many(handles)
    mgr.synchronize()
    for h in handles:
        h.free()
    for c, want, old in zip(new_caches, rows, id_lists):
        new_ids = c.page_table.retrieve().numpy()
        assert len(new_ids) == len(old)
        assert c.isswap[: len(new_ids)].tolist() == (new_ids >= main).tolist()
        swap_ops.reload_rows(ref, new_ids, want)
    assert torch.equal(pool.pages.cpu().view(torch.uint8), ref.view(torch.uint8))
    assert chunks.available_ids[-1] == [0]  # every chunk merged back


def test_single_task_reference_api():
    L, ps, hkv, d = 2, 8, 8, 128
    pool = dk.VirtualPagePool(L, 12, 2, ps, DEV, torch.float16)
    ref = _fill(pool, 6)
    pta = dk.PageTableAllocator(4, 1024, ps, DEV)
    chunks = dk.CpuChunkPool(L, 4, ps, torch.float16)
    mgr = dk.KVCacheManager(pool, chunks, pta)
    c = dk.VirtualPagedKVCache.empty(pta, pool)
    c.extend(3 * ps)
    old = c.page_table.retrieve().numpy().copy()
    h = mgr.copy_gpu_to_cpu(c, "task")
    c.free()
    c2 = mgr.copy_cpu_to_gpu(h, "task")
    mgr.synchronize()
    h.free()
    new = c2.page_table.retrieve().numpy()
    assert not np.array_equal(old, new)
    got = pool.pages.cpu()
    assert torch.equal(got[:, torch.as_tensor(new, dtype=torch.long)].view(torch.uint8),
                       ref[:, torch.as_tensor(old, dtype=torch.long)].view(torch.uint8))


@pytest.mark.parametrize("staging_mib", [None, 24])
def test_back_to_back_offloads_then_reloads_share_the_staging_buffer(staging_mib):
    """The reference offloads and reloads task by task in a loop
    (deserve_worker/engine/microbatch/processor.py:62-88). Here every such call is
    asynchronous and all of them go through one staging buffer, so consecutive calls
    with NO host wait in between must order themselves on the device: a task is
    large enough (64 MiB) that its DMA is still running when the next call's pack
    kernel (or host->device burst) wants the same staging half."""
    L, ps, hkv, d = 8, 16, 8, 128
    n_tasks, n_pages = 4, 128
    dtype = torch.bfloat16
    pool = dk.VirtualPagePool(L, 2 * n_tasks * n_pages + 8, 0, ps, DEV, dtype, n_kv_heads=hkv, head_dim=d)
    g = torch.Generator(device=DEV).manual_seed(11)
    pool.pages.normal_(0.0, 1.0, generator=g)
    pta = dk.PageTableAllocator(2 * n_tasks, n_pages * ps, ps, DEV)
    chunks = dk.CpuChunkPool(L, 10, ps, dtype, n_kv_heads=hkv, head_dim=d)  # 512 page rows of every layer
    mgr = dk.KVCacheManager(pool, chunks, pta, staging_bytes=None if staging_mib is None else staging_mib << 20)
    caches = []
    for _ in range(n_tasks):
        c = dk.VirtualPagedKVCache.empty(pta, pool)
        c.extend(n_pages * ps)
        caches.append(c)
    id_lists = [c.page_table.retrieve().numpy().copy() for c in caches]
    ref = pool.pages.cpu()
    handles = [mgr.copy_gpu_to_cpu(c, f"t{i}") for i, c in enumerate(caches)]  # no wait in between
    mgr.synchronize()
    rows = [swap_ops.offload_rows(ref, ids) for ids in id_lists]
    for h, want in zip(handles, rows):
        assert torch.equal(h.retrieve()[: n_pages * L].view(torch.uint8), want.view(torch.uint8))
    for c in caches:
        c.free()
    pool.pages.fill_(-3.0)
    filler = dk.VirtualPagedKVCache.empty(pta, pool)
    filler.extend(5 * ps)  # shifts the ids the reloads get
    ref = pool.pages.cpu()
    new_caches = [mgr.copy_cpu_to_gpu(h, f"t{i}") for i, h in enumerate(handles)]  # no wait in between
    mgr.synchronize()
    for c, want in zip(new_caches, rows):
        swap_ops.reload_rows(ref, c.page_table.retrieve().numpy(), want)
    assert torch.equal(pool.pages.cpu().view(torch.uint8), ref.view(torch.uint8))


def test_pack_skips_page_ids_outside_the_pool_and_reports_them():
    """An id >= num_pages (a stale table entry) or < 0 touches no memory: the row
    is skipped, the other rows are copied, and the status word reads 1 (bad page
    id). The check replaces the access; nothing faults."""
    L, P, ps, hkv, d = 2, 12, 16, 2, 64
    pool = dk.GpuPagePool(L, P, ps, DEV, torch.bfloat16, n_kv_heads=hkv, head_dim=d)
    ref = _fill(pool, 9)
    ids_host = np.array([3, P + 5, 7, -2, 0], dtype=np.int32)
    ids = torch.from_numpy(ids_host).to(DEV)
    indptr = torch.tensor([0, len(ids_host)], dtype=torch.int32, device=DEV)
    packed = torch.zeros(len(ids_host) * L, *pool.pages.shape[2:], dtype=torch.bfloat16, device=DEV)
    _lib.check(_lib.lib.dsv_pack_pages(pool.pages.data_ptr(), pool.layer_stride_bytes, pool.page_bytes, P,
                                       ids.data_ptr(), indptr.data_ptr(), 1, len(ids_host), 0, L, packed.data_ptr(),
                                       _lib.current_stream_ptr(DEV)))
    assert _lib.read_device_status() == 1
    got = packed.cpu().view(L, len(ids_host), *pool.pages.shape[2:])
    for j, pid in enumerate(ids_host.tolist()):
        if 0 <= pid < P:
            assert torch.equal(got[:, j], ref[:, pid])
        else:
            assert not got[:, j].any()
    # the scatter direction: rows with a bad id leave the pool untouched
    before = pool.pages.cpu()
    _lib.check(_lib.lib.dsv_unpack_pages(packed.data_ptr(), pool.pages.data_ptr(), pool.layer_stride_bytes,
                                         pool.page_bytes, P, ids.data_ptr(), indptr.data_ptr(), 1, len(ids_host), 0, L,
                                         _lib.current_stream_ptr(DEV)))
    assert _lib.read_device_status() == 1
    assert torch.equal(pool.pages.cpu().view(torch.uint8), before.view(torch.uint8))
