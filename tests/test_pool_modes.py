"""The fast pool's two modes: one allocation managed by an offset allocator ("slab"), and a paged virtual range of twice
the size whose pages come from a physical budget ("vmm").  The host backends carry the page bookkeeping without a driver,
so the mode's logic is tested here; the CUDA side maps real pages (GPU test)."""
import pytest

from chains import train_chain
from dataflow_b200.core import from_sim_chain
from dataflow_b200.runtime import Engine, FakeBackend, PoolProbe
from dataflow_b200.sim import run
from dataflow_b200.sim.policies.pressurefit import pressurefit

MB = 1 << 20


def fragment(pool):
    """Eight 8 MiB blocks, every other one freed: 32 MiB free, no hole larger than 8 MiB."""
    blocks = [pool.get(8 * MB) for _ in range(8)]
    assert not any(b[2] for b in blocks)
    for b in blocks[::2]:
        pool.put(b[0])
    return blocks[1::2]


def test_fragmentation_overflows_one_allocation_but_not_the_paged_range():
    slab = PoolProbe(FakeBackend(), 64 * MB, vm=False)
    fragment(slab)
    assert slab.get(30 * MB)[2] is True and slab.stats()["overflows"] == 1            # no contiguous 30 MiB
    vm = PoolProbe(FakeBackend(), 64 * MB, vm=True)
    fragment(vm)
    h, ptr, overflow = vm.get(30 * MB)
    st = vm.stats()
    assert overflow is False and st["overflows"] == 0 and st["mode"] == "vmm"
    assert st["va_bytes"] == 128 * MB and st["phys_pages"] == 32
    assert st["held_pages"] == 31 and st["mapped_pages"] <= st["phys_pages"]
    assert st["reclaims"] == 15                      # the freed blocks' pages moved under the new block


def test_paged_range_never_exceeds_its_physical_budget():
    vm = PoolProbe(FakeBackend(), 64 * MB, vm=True)
    kept = fragment(vm)
    big = vm.get(30 * MB)
    more = vm.get(8 * MB)                            # 31 pages held + 4 > 32: a real out-of-memory, counted as an overflow
    assert more[2] is True and vm.stats()["overflows"] == 1 and vm.stats()["held_pages"] == 31
    vm.put(big[0])
    again = vm.get(8 * MB)
    assert again[2] is False and vm.stats()["mapped_pages"] <= 32
    for b in kept:
        vm.put(b[0])
    assert vm.stats()["held_pages"] == 4


def test_repeating_the_same_allocations_maps_nothing_new():
    """Pages nobody holds stay mapped: a steady-state step that allocates the same sizes in the same order costs no page work."""
    vm = PoolProbe(FakeBackend(), 64 * MB, vm=True)

    def step():
        a = [vm.get(5 * MB) for _ in range(6)]
        b = vm.get(20 * MB)
        for x in a:
            vm.put(x[0])
        c = vm.get(24 * MB)
        vm.put(b[0])
        vm.put(c[0])
    step()
    first = vm.stats()["maps"]
    for _ in range(3):
        step()
    assert vm.stats()["maps"] == first and vm.stats()["overflows"] == 0


def test_small_blocks_share_pages():
    vm = PoolProbe(FakeBackend(), 8 * MB, vm=True)
    small = [vm.get(4096) for _ in range(100)]
    assert vm.stats()["held_pages"] == 1
    for s in small[:-1]:
        vm.put(s[0])
    assert vm.stats()["held_pages"] == 1             # the last block still holds the page
    vm.put(small[-1][0])
    assert vm.stats()["held_pages"] == 0


@pytest.mark.parametrize("cap", [6000, 2200])
def test_engine_on_a_paged_pool_reproduces_the_simulator(cap):
    r = pressurefit(train_chain(), cap)
    log = run(r.chain)
    prog = from_sim_chain(r.chain)
    eng = Engine(FakeBackend())
    eng.session.native.ensure_pools(cap + 4 * MB, 10 ** 7, 0.0, True)
    assert eng.session.native.fast_pool_stats()["mode"] == "vmm"
    res = eng.execute(prog, manage_pools=False).raise_if_failed()
    assert res.slab_overflows == 0 and res.makespan_us == log.makespan


@pytest.mark.gpu
def test_cuda_pages_are_mapped_moved_and_usable():
    """Real pages: write through a block, fragment, allocate a block larger than any hole, write and read it back."""
    import torch
    from dataflow_b200.ops import native
    from dataflow_b200.runtime import CudaBackend
    be = CudaBackend(0, "poll")
    vm = PoolProbe(be, 64 * MB, vm=True)
    assert vm.stats()["mode"] == "vmm"
    kept = fragment(vm)
    views = []
    for i, (h, ptr, ov) in enumerate(kept):
        t = native().tensor_from_ptr(ptr, [8 * MB // 4], "fp32", 0)
        t.fill_(float(i + 1))
        views.append(t)
    h, ptr, overflow = vm.get(30 * MB)
    assert overflow is False and vm.stats()["reclaims"] > 0
    big = native().tensor_from_ptr(ptr, [30 * MB // 4], "fp32", 0)
    big.copy_(torch.arange(big.numel(), device="cuda", dtype=torch.float32))
    torch.cuda.synchronize()
    assert float(big[-1]) == float(big.numel() - 1) and float(big[12345]) == 12345.0
    for i, t in enumerate(views):                    # the kept blocks were not disturbed by the page moves
        assert float(t.min()) == float(i + 1) == float(t.max())
    del big, views, t
    torch.cuda.synchronize()
    vm.put(h)
    for b in kept:
        vm.put(b[0])
    assert vm.stats()["held_pages"] == 0
