"""Index arithmetic of the down projection's epilogue (k_prefill_gemm, llmxabe_b200/csrc/prefill_kernels.cuh),
checked on the CPU: an epilogue warp turns 32 tokens x 16 outputs around in 2 KB of shared memory so that
four lanes store 64 neighbouring bytes of one result row.  Lane = token writes its 16 outputs as four
16-byte chunks, chunk c at position c ^ ((lane / 2) % 4) of its 64-byte row; pass `it` of the read-back
gives lane l chunk l % 4 of token row it * 8 + l / 4.  The test checks that every value comes back where
it belongs and that neither side has a shared-memory bank conflict (a 16-byte access is served a
quarter-warp at a time: its eight lanes must cover all 32 banks)."""
import numpy as np


def _store_addresses():
    lane = np.arange(32)[:, None]
    c = np.arange(4)[None, :]
    return lane * 16 + ((c ^ ((lane >> 1) & 3)) << 2)          # float index of chunk c of lane's row


def _load_addresses(it: int):
    lane = np.arange(32)
    row, c = it * 8 + (lane >> 2), lane & 3
    return row, c, row * 16 + ((c ^ ((row >> 1) & 3)) << 2)


def test_every_output_comes_back_at_its_row_and_column():
    stage = np.full(32 * 16, -1, dtype=np.int64)
    st = _store_addresses()
    for lane in range(32):
        for c in range(4):
            for k in range(4):
                stage[st[lane, c] + k] = lane * 16 + c * 4 + k   # token lane, output 4 c + k
    assert (stage >= 0).all()
    seen = set()
    for it in range(4):
        row, c, addr = _load_addresses(it)
        for lane in range(32):
            for k in range(4):
                assert stage[addr[lane] + k] == row[lane] * 16 + c[lane] * 4 + k
                seen.add((int(row[lane]), int(c[lane]) * 4 + k))
    assert len(seen) == 32 * 16


def _banks_of_quarter(addr_floats):
    banks = []
    for a in addr_floats:
        banks.extend(((a + k) % 32) for k in range(4))
    return banks


def test_neither_side_has_a_bank_conflict():
    st = _store_addresses()
    for c in range(4):                                           # one 16-byte store instruction per chunk
        for q in range(4):                                       # quarter-warps
            banks = _banks_of_quarter(st[8 * q:8 * q + 8, c])
            assert sorted(banks) == list(range(32)), (c, q)
    for it in range(4):
        _, _, addr = _load_addresses(it)
        for q in range(4):
            banks = _banks_of_quarter(addr[8 * q:8 * q + 8])
            assert sorted(banks) == list(range(32)), (it, q)
