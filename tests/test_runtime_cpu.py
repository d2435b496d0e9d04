"""Host-side pieces of the C ABI that make no CUDA call: the packed-int4 container, the
MatMulNBits nibble convention in both directions, the prepack gates, the empty weight table
and the operator counters. CPU only."""
import numpy as np
import pytest

import yscv_b200
from yscv_b200 import lib as binding


def test_container_round_trip(oracle):
    n, k, g = 24, 96, 32
    rng = np.random.default_rng(5)
    packed, scales = oracle.pack_int4(rng.normal(0, 0.02, n * k).astype(np.float32), n, k, g)
    blob = yscv_b200.int4_container_write(packed, scales, n, k, g)
    assert len(blob) == 64 + (n * k // 2 + 15) // 16 * 16 + n * (k // g) * 4
    assert blob[:8] == b"YSCVINT4"
    p2, s2, n2, k2, g2 = yscv_b200.int4_container_read(blob)
    assert (n2, k2, g2) == (n, k, g)
    assert np.array_equal(p2, packed) and np.array_equal(s2, scales)


def test_container_rejects_damage(oracle):
    packed, scales = oracle.pack_int4(np.ones(8 * 64, np.float32), 8, 64, 32)
    blob = bytearray(yscv_b200.int4_container_write(packed, scales, 8, 64, 32))
    for bad in (bytes(blob[:40]),                      # shorter than the header
                bytes(blob[:-4]),                      # scales cut short
                b"NOTACONT" + bytes(blob[8:]),         # wrong magic
                bytes(blob[:8]) + (7).to_bytes(4, "little") + bytes(blob[12:])):  # unknown version
        with pytest.raises(yscv_b200.YscvCudaError):
            yscv_b200.int4_container_read(bad)
    # header that contradicts itself: k no longer a multiple of the group size
    broken = bytearray(blob)
    broken[24:32] = (65).to_bytes(8, "little")
    with pytest.raises(yscv_b200.YscvCudaError):
        yscv_b200.int4_container_read(bytes(broken))
    # odd group size at write time
    with pytest.raises(yscv_b200.YscvCudaError):
        yscv_b200.int4_container_write(packed, scales, 8, 64, 0)


def test_matmulnbits_export_inverts_import(oracle):
    src = np.arange(256, dtype=np.uint8)
    there = yscv_b200.int4_to_matmulnbits(src)
    assert np.array_equal(yscv_b200.int4_from_matmulnbits(there), src)
    # exported nibbles are q + 8 of the sign-extended nibbles
    for s, u in zip(src.tolist(), there.tolist()):
        assert (u & 15) == oracle.lib.yo_unpack_low(s) + 8
        assert (u >> 4) == oracle.lib.yo_unpack_high(s) + 8


def test_prepack_gates_follow_the_reference():
    lib = yscv_b200.load_library()
    # should_prepack_i8_b (plan/build.rs:1371-1377): (k >= 4 && n % 16 == 0) || (k >= 512 && n >= 1024)
    for k, n in [(4, 16), (3, 16), (4, 17), (512, 1024), (512, 1030), (511, 1030), (1024, 1000)]:
        want = (k >= 4 and n % 16 == 0) or (k >= 512 and n >= 1024)
        assert bool(lib.yscv_cuda_should_prepack_i8_b(k, n)) == want, (k, n)
    # should_use_prepacked_i8_b (runner/layout.rs:6-11)
    for m, k, n in [(4, 4, 32), (3, 4, 32), (4, 4, 33), (64, 512, 1024), (65, 512, 1030), (1, 512, 1030), (1, 8, 64)]:
        want = (m >= 4 and k >= 4 and n >= 32 and n % 16 == 0) or (m <= 64 and k >= 512 and n >= 1024)
        assert bool(lib.yscv_cuda_should_use_prepacked_i8_b(m, k, n)) == want, (m, k, n)


def test_empty_registry():
    reg = yscv_b200.Registry()
    assert len(reg) == 0
    assert reg.get_int4("model.layers.0.mlp.down_proj.weight") is None
    assert reg.get_i8b("absent") is None
    reg.close()


def test_quant_stats_start_at_zero_and_have_no_cpu_fallback():
    yscv_b200.quant_stats_reset()
    st = yscv_b200.quant_stats()
    assert set(st) == {n for n, _ in binding.QuantStats._fields_}
    assert all(v == 0 for v in st.values())
