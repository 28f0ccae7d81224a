"""Shared-memory ring: slot lifecycle, stale generations, slow readers, abort (spawned readers,
the technique of the reference's tests/test_ring.py:21-63)."""

import multiprocessing as mp
import os
import stat

import pytest

from ep_xpress_b200 import native


@pytest.fixture()
def ring_path(tmp_path):
    return str(tmp_path / "unit.ring")


def test_lifecycle_and_masks(ring_path):
    m = native.load()
    ring = m.HostRing(ring_path, 2, 1000, True)
    assert (ring.slots(), ring.slot_bytes()) == (2, 1000)
    assert stat.S_IMODE(os.stat(ring_path).st_mode) == 0o600
    a = ring.try_claim(7, 0b110)
    b = ring.try_claim(8, 0b010)
    assert {a, b} == {0, 1} and ring.try_claim(9, 0b010) == -1          # bounded: both slots in use
    assert ring.ready(a, 7) == -1                                       # not published yet
    ring.payload(a)[:3] = 5
    ring.publish(a, 3)
    peer = m.HostRing(ring_path)
    assert peer.ready(a, 7) == 3 and peer.ready(a, 8) == -1             # stale/other generations never match
    assert peer.payload(a)[:3].tolist() == [5, 5, 5]
    assert peer.ack(a, 7, 1) is False                                   # rank 2 has not read yet
    with pytest.raises(RuntimeError, match="duplicate"):
        peer.ack(a, 7, 1)
    with pytest.raises(RuntimeError, match="not an expected reader"):
        peer.ack(a, 7, 0)
    assert ring.try_claim(9, 0b010) == -1                               # slow reader blocks only its slot
    assert peer.ack(a, 7, 2) is True
    with pytest.raises(RuntimeError, match="stale"):
        peer.ack(a, 7, 2)
    assert ring.try_claim(9, 0b010) == a                                # slot reusable
    with pytest.raises(ValueError):
        ring.try_claim(10, 0)
    with pytest.raises(IndexError):
        ring.ready(5, 1)


def test_abort_is_sticky_and_visible(ring_path):
    m = native.load()
    ring = m.HostRing(ring_path, 1, 64, True)
    peer = m.HostRing(ring_path)
    assert not peer.aborted()
    ring.abort()
    assert peer.aborted()
    with pytest.raises(RuntimeError, match="aborted"):
        peer.ready(0, 1)
    with pytest.raises(RuntimeError, match="aborted"):
        ring.try_claim(1, 1)
    ring.close()
    with pytest.raises(RuntimeError, match="closed"):
        ring.slots()


def test_rejects_foreign_files(tmp_path):
    m = native.load()
    bogus = tmp_path / "bogus.ring"
    bogus.write_bytes(b"\0" * 8192)
    with pytest.raises(RuntimeError, match="magic"):
        m.HostRing(str(bogus))
    with pytest.raises(RuntimeError):
        m.HostRing(str(tmp_path / "missing.ring"))


def _reader(path, rank, chunks, delay, out):
    import time
    m = native.load()
    ring = m.HostRing(path)
    total = 0
    for generation in range(chunks):
        while True:
            hit = [s for s in range(ring.slots()) if ring.ready(s, generation) >= 0]
            if hit:
                break
            time.sleep(0.0005)
        total += int(ring.payload(hit[0])[0])
        if delay:
            time.sleep(delay)
        ring.ack(hit[0], generation, rank)
    out.put((rank, total))


def test_stream_of_chunks_through_two_slots_with_a_slow_reader(ring_path):
    m = native.load()
    chunks = 32
    ring = m.HostRing(ring_path, 2, 256, True)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    readers = [ctx.Process(target=_reader, args=(ring_path, rank, chunks, 0.002 if rank == 2 else 0, out))
               for rank in (1, 2)]
    for p in readers:
        p.start()
    import time
    deadline = time.monotonic() + 60
    for generation in range(chunks):
        while True:
            slot = ring.try_claim(generation, 0b110)
            if slot >= 0:
                break
            assert time.monotonic() < deadline
            time.sleep(0.0005)
        ring.payload(slot)[0] = generation % 200
        ring.publish(slot, 1)
    results = dict(out.get(timeout=60) for _ in readers)
    for p in readers:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert results == {1: sum(g % 200 for g in range(chunks)), 2: sum(g % 200 for g in range(chunks))}
