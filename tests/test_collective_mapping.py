"""Index arithmetic of the chunked peer all-reduce (csrc/peer_collectives.cu::allreduce_kernel),
restated on the CPU.

The kernel synchronises block b of every rank with block b of the other ranks only. That is enough
exactly when the thread that reads element j of a chunk in the collect phase has the same global
thread index as the thread that reduced it on the owner rank. These cases pin that invariant for
chunk sizes that are not multiples of the grid's thread count, where an index-by-absolute-position
mapping pairs a reader with a writer of a different block."""
import pytest

THREADS = 512
UNROLL = 4


def _writer_thread(j: int, nthreads: int) -> int:
    """Global thread index that handles chunk-relative element j in phase 1 (strided loop, unrolled)."""
    # i0 = tid + k * nthreads * UNROLL, i = i0 + u * nthreads  =>  i mod nthreads == tid
    return j % nthreads


def _reader_thread(j: int, nthreads: int) -> int:
    """Global thread index that reads chunk-relative element j of any owner's chunk in phase 2."""
    return j % nthreads


def _old_reader_thread(owner: int, chunk: int, j: int, nthreads: int) -> int:
    """The mapping the kernel must NOT use: thread chosen by the absolute position in the buffer."""
    return (owner * chunk + j) % nthreads


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("blocks", [8, 32, 64, 128])
@pytest.mark.parametrize("n_elems", [(1 << 22) + 24, 3 * 1000 * 1000 + 8, 16384 * 8])
def test_reader_and_writer_share_a_block(world, blocks, n_elems):
    vec = 8                                     # bf16 elements per 16-byte vector
    unit = vec * world
    n_pad = (n_elems + unit - 1) // unit * unit
    nvec = n_pad // vec
    chunk = nvec // world
    nthreads = blocks * THREADS
    assert chunk * world == nvec
    step = max(1, chunk // 997)                 # sample the chunk, always including its ends
    for owner in range(world):
        for j in list(range(0, chunk, step)) + [chunk - 1]:
            w, r = _writer_thread(j, nthreads), _reader_thread(j, nthreads)
            assert w // THREADS == r // THREADS
    if chunk % nthreads:
        # the position-based mapping breaks the invariant for these sizes
        bad = sum(_old_reader_thread(1, chunk, j, nthreads) // THREADS != _writer_thread(j, nthreads) // THREADS
                  for j in range(0, chunk, step))
        assert bad > 0


def test_unrolled_loop_covers_every_element_once():
    """tid + k * nthreads * U + u * nthreads enumerates [0, chunk) exactly once."""
    for chunk, nthreads in [(1000, 64), (4097, 512), (12345, 1024)]:
        seen = [0] * chunk
        for tid in range(nthreads):
            i0 = tid
            while i0 < chunk:
                for u in range(UNROLL):
                    i = i0 + u * nthreads
                    if i < chunk:
                        seen[i] += 1
                        assert i % nthreads == tid
                i0 += nthreads * UNROLL
        assert all(c == 1 for c in seen)
