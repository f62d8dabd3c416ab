"""CPU: an executable model of the synchronisation protocol of the in-switch exchange that is fused into the last GEMM of the
tensor-parallel FFN block (pyc_b200/csrc/gemm_fp8.cu, SWITCH_REDUCE): threads stand in for the epilogue warps, the
publisher warp and the reducer warp of every CTA of every rank; shared Python lists stand in for the flag words in the
receivers' memory.  What the model checks is the protocol's logic, not the CUDA code:
  * epochs: a reducer never consumes a partial sum of an EARLIER call, although flag words and data buffers are reused;
  * the epilogue-to-publisher hand-off is a monotonic counter, so a publisher that is several tiles behind (its fence is
    slower than a tile) still publishes every tile exactly once -- the two-phase barrier it replaced could not;
  * every rank leaves a call only after every rank's reducers have finished (the "fin" rendezvous), so the next call may
    overwrite the partial sums.
"""
import random
import threading
import time

WORLD, CTAS, TILES_PER_CTA, CALLS = 4, 3, 6, 4
TILES = CTAS * TILES_PER_CTA


class Machine:
    def __init__(self):
        self.partial = [[None] * TILES for _ in range(WORLD)]                 # [rank][tile] = (call, rank) once stored
        self.flags = [[[0] * WORLD for _ in range(TILES)] for _ in range(WORLD)]   # [receiver][tile][sender] = epoch
        self.fin = [[[0] * WORLD for _ in range(CTAS)] for _ in range(WORLD)]      # [receiver][cta][sender] = epoch
        self.epochs = [[0] * CTAS for _ in range(WORLD)]                      # local counters, advanced by the kernel itself
        self.errors = []


def wait_until(cond, what, errors, limit=20.0):
    t0 = time.monotonic()
    while not cond():
        if time.monotonic() - t0 > limit:
            errors.append(f"bounded wait ran out: {what}")
            return False
        time.sleep(0)
    return True


def cta_call(m, rank, cta, call, rng):
    """One CTA of one rank during one call: epilogue, publisher and reducer run concurrently."""
    epoch = m.epochs[rank][cta] + 1
    tiles = [cta + i * CTAS for i in range(TILES_PER_CTA)]                    # the persistent schedule, same on every rank
    stored = [0]                                                              # shared-memory counter of stored tiles

    def epilogue():
        for t in tiles:
            time.sleep(rng.random() * 0.0004)                                 # a tile of the GEMM
            m.partial[rank][t] = (call, rank)                                 # this rank's partial sum of the tile
            stored[0] += 1                                                    # red.release.cta on the counter

    def publisher():
        published = 0
        while published < len(tiles):
            done = stored[0]                                                  # ld.acquire.cta
            if done > published:
                time.sleep(0.0015)                                            # the system-scope fence: slower than a tile
                for t in tiles[published:done]:
                    for peer in range(WORLD):
                        m.flags[peer][t][rank] = epoch                        # single writer per word
                published = done
            else:
                time.sleep(0)

    def reducer():
        for t in tiles:
            if not wait_until(lambda: all(m.flags[rank][t][s] - epoch >= 0 for s in range(WORLD)), f"flags of tile {t}", m.errors):
                return
            for s in range(WORLD):                                            # multimem.ld_reduce reads every rank's partial sum
                if m.partial[s][t] != (call, s):
                    m.errors.append(f"rank {rank} call {call} tile {t}: read {m.partial[s][t]} from rank {s}")
        for peer in range(WORLD):
            m.fin[peer][cta][rank] = epoch
        wait_until(lambda: all(m.fin[rank][cta][s] - epoch >= 0 for s in range(WORLD)), f"fin of cta {cta}", m.errors)

    threads = [threading.Thread(target=f) for f in (epilogue, publisher, reducer)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    m.epochs[rank][cta] = epoch                                               # thread 0 after the CTA's warps have met


def rank_main(m, rank, seed):
    rng = random.Random(seed)
    for call in range(CALLS):
        ctas = [threading.Thread(target=cta_call, args=(m, rank, c, call, rng)) for c in range(CTAS)]
        for th in ctas:
            th.start()
        for th in ctas:
            th.join()                                                         # the kernel ends when all its CTAs have
        time.sleep(rng.random() * 0.002)                                      # host jitter before the next call


def test_epochs_counter_handoff_and_fin_rendezvous_hold_under_lag_and_jitter():
    m = Machine()
    ranks = [threading.Thread(target=rank_main, args=(m, r, 1000 + r)) for r in range(WORLD)]
    for th in ranks:
        th.start()
    for th in ranks:
        th.join(timeout=120)
        assert not th.is_alive(), "a rank did not finish"
    assert m.errors == []
    assert all(e == CALLS for row in m.epochs for e in row)
    assert all(m.flags[r][t][s] == CALLS for r in range(WORLD) for t in range(TILES) for s in range(WORLD))
