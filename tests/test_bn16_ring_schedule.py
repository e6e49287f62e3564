"""The chunk schedule of the bf16 batch-norm kernels' copy ring (``csrc/bn_nhwc_bf16.cu``: ``bn16_plan`` and
``bn16_stream``) restated on the CPU: chunk sizes, which chunk lands in which slot under which barrier phase, and
the thread-to-channel mapping that lets a thread keep its channels' constants in registers."""
import itertools

STAGE = 16384
THREADS = 256


def plan(total_bytes, per_sm, sms=148):
    cap = per_sm * sms
    ch = STAGE
    while ch > 4096 and (total_bytes + ch - 1) // ch < 4 * cap:
        ch >>= 1
    grid = min((total_bytes + ch - 1) // ch, cap)
    return max(grid, 1), ch


def cta_schedule(total_bytes, ch, grid, block, stages, reverse):
    """Events of one CTA in program order: ('issue', chunk, slot, phase) / ('consume', chunk, slot, phase)."""
    n_chunks = (total_bytes + ch - 1) // ch
    n_mine = (n_chunks - block + grid - 1) // grid if block < n_chunks else 0

    def chunk_of(it):
        k = block + it * grid
        return n_chunks - 1 - k if reverse else k

    ev = [("issue", chunk_of(it), it % stages, (it // stages) & 1) for it in range(min(stages, n_mine))]
    for it in range(n_mine):
        ev.append(("consume", chunk_of(it), it % stages, (it // stages) & 1))      # wait on the slot's phase, then a CTA barrier
        if it >= 1 and it - 1 + stages < n_mine:
            nxt = it - 1 + stages
            ev.insert(len(ev) - 1, ("issue", chunk_of(nxt), nxt % stages, (nxt // stages) & 1))
    return ev, n_chunks


def test_every_chunk_is_copied_and_consumed_once_and_slots_are_never_overwritten_early():
    for (p, c), per_sm, stages, reverse in itertools.product(
            [(128 * 112 * 112, 64), (6272, 2048), (315, 1024), (2, 64), (25088, 256)], (2, 3), (2, 3, 4), (False, True)):
        total = p * c * 2
        grid, ch = plan(total, per_sm)
        assert ch % (2 * c) == 0 and ch in (4096, 8192, 16384) and grid <= 4 * 148
        seen = []
        for block in range(grid):
            ev, n_chunks = cta_schedule(total, ch, grid, block, stages, reverse)
            in_slot = {}
            for kind, chunk, slot, phase in ev:
                assert 0 <= chunk < n_chunks
                if kind == "issue":
                    assert slot not in in_slot, "slot refilled before its chunk was consumed"
                    in_slot[slot] = (chunk, phase)
                else:
                    assert in_slot.pop(slot) == (chunk, phase)
                    seen.append(chunk)
            assert not in_slot
        assert sorted(seen) == list(range(n_chunks))
        # the last chunk may be short but is a whole number of 16-byte pieces and of rows
        tail = total - (n_chunks - 1) * ch
        assert 0 < tail <= ch and tail % 16 == 0 and tail % (2 * c) == 0


def test_a_thread_always_meets_the_same_eight_channels():
    for c in (8, 64, 256, 1024, 2048):
        tpr = c // 8
        assert THREADS % tpr == 0
        for ch in (4096, 8192, 16384):
            for chunk_start in (0, ch, 7 * ch):
                for tid in (0, 1, tpr - 1, 37 % THREADS, 255):
                    cols = set()
                    for m in range(STAGE // 16 // THREADS):
                        byte = chunk_start + (m * THREADS + tid) * 16
                        if (m * THREADS + tid) * 16 < ch:
                            cols.add((byte // 2) % c)
                    assert cols == {(tid % tpr) * 8}
