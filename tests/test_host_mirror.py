"""The host mirror of oxmera-core / oxmera-tensor / oxmera-runtime against the
hand cases of the reference's exercise specs A1, A2, A3 and A5.  Storage is
served by a host-memory stand-in backend, so no GPU is needed."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Device, Layout, Tensor

HAND = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "a4_hand_cases.json")))


class HostStandIn:
    """Implements only the storage plumbing Tensor needs, in host memory."""

    def __init__(self):
        self.bufs = {}

    def device(self):
        return Device.cuda(0)

    def name(self):
        return "host-stand-in"

    def _alloc(self, nbytes):
        buf = C.create_string_buffer(max(nbytes, 16))
        self.bufs[C.addressof(buf)] = buf
        return C.addressof(buf)

    def _free(self, ptr):
        self.bufs.pop(ptr, None)

    def _h2d(self, dst, src, n):
        C.memmove(dst, src, n)

    def _d2h(self, dst, src, n):
        C.memmove(dst, src, n)

    def synchronize(self):
        pass

    def _materialize(self, t):
        host = t.to_host()
        return Tensor.from_host(host, t.shape, t.dtype, self)


@pytest.fixture()
def be():
    return HostStandIn()


def t23(be):
    return Tensor.from_host(np.array([1, 2, 3, 4, 5, 6], np.float32), (2, 3), DType.F32, be)


# ---- A1: exercises/a1-shape-and-strides/tests/spec.rs:11-93 ----
def test_dtype_sizes_and_classes():
    assert [d.size_in_bytes() for d in (DType.F32, DType.F64, DType.I32, DType.I64, DType.U8, DType.Bool)] == [4, 8, 4, 8, 1, 1]
    assert DType.BF16.size_in_bytes() == 2 and DType.F16.size_in_bytes() == 2
    assert DType.F32.is_float() and DType.F64.is_float() and DType.BF16.is_float() and DType.F16.is_float()
    assert not any(d.is_float() for d in (DType.I32, DType.I64, DType.U8, DType.Bool))


def test_numel_hand_cases():
    assert ox.numel(()) == 1 and ox.numel((0,)) == 0 and ox.numel((2, 3)) == 6
    assert ox.numel((2, 0, 3)) == 0 and ox.numel((1, 1, 1)) == 1


def test_contiguous_strides_hand_cases():
    assert ox.contiguous_strides(()) == ()
    assert ox.contiguous_strides((4,)) == (1,)
    assert ox.contiguous_strides((2, 3)) == (3, 1)
    assert ox.contiguous_strides((2, 1, 3)) == (3, 3, 1)
    assert ox.contiguous_strides((4, 2, 3)) == (6, 3, 1)


def test_offset_of_hand_cases():
    l = Layout.contiguous((2, 3))
    assert [l.offset_of(i) for i in ([0, 0], [0, 2], [1, 0], [1, 2])] == [0, 2, 3, 5]
    assert Layout.contiguous(()).offset_of([]) == 0
    for bad in ([0], [0, 0, 0]):
        with pytest.raises(ox.RankMismatch):
            l.offset_of(bad)
    for bad in ([2, 0], [0, 3]):
        with pytest.raises(ox.IndexOutOfBounds):
            l.offset_of(bad)


def test_contiguity_hand_cases():
    assert Layout.contiguous((2, 3)).is_contiguous()
    assert Layout.contiguous(()).is_contiguous()
    assert Layout.contiguous((0, 3)).is_contiguous()
    assert not Layout((2, 3), (1, 2), 0).is_contiguous()


def test_contiguous_offsets_are_a_bijection():
    rng = np.random.default_rng(0)
    for _ in range(50):
        dims = tuple(int(x) for x in rng.integers(1, 4, size=rng.integers(0, 4)))
        l = Layout.contiguous(dims)
        seen = {l.offset_of(list(idx)) for idx in np.ndindex(*dims)}
        assert seen == set(range(ox.numel(dims)))


# ---- A2: exercises/a2-broadcasting/tests/spec.rs:15-54 ----
@pytest.mark.parametrize("case", HAND["broadcast_ok"]["cases"], ids=str)
def test_broadcast_hand_cases(case):
    assert list(ox.broadcast_shapes(case[0], case[1])) == case[2]


@pytest.mark.parametrize("case", HAND["broadcast_refuse"]["cases"], ids=str)
def test_broadcast_refusals_carry_the_operands(case):
    with pytest.raises(ox.BroadcastIncompatible) as e:
        ox.broadcast_shapes(case[0], case[1])
    assert (list(e.value.lhs), list(e.value.rhs)) == (case[0], case[1])


def test_broadcast_is_commutative_and_idempotent():
    rng = np.random.default_rng(1)
    for _ in range(200):
        a = tuple(int(x) for x in rng.integers(0, 4, size=rng.integers(0, 4)))
        b = tuple(int(x) for x in rng.integers(0, 4, size=rng.integers(0, 4)))
        try:
            ab = ox.broadcast_shapes(a, b)
        except ox.BroadcastIncompatible:
            with pytest.raises(ox.BroadcastIncompatible):
                ox.broadcast_shapes(b, a)
            continue
        assert ab == ox.broadcast_shapes(b, a)
        assert ox.broadcast_shapes(a, a) == a and ox.broadcast_shapes(a, ()) == a


# ---- A3: exercises/a3-strided-views/tests/spec.rs:17-92 ----
def test_permute_reads_the_transpose_and_shares_storage(be):
    t = t23(be)
    tt = t.permute([1, 0])
    assert tt.shape == (3, 2)
    assert [tt.get_f32(i) for i in ([0, 0], [0, 1], [1, 0], [2, 1])] == [1.0, 4.0, 2.0, 6.0]
    assert tt.storage() is t.storage()


def test_narrow_windows_the_middle_and_shares_storage(be):
    t = t23(be)
    n = t.narrow(1, 1, 2)
    assert n.shape == (2, 2)
    assert [n.get_f32(i) for i in ([0, 0], [0, 1], [1, 0], [1, 1])] == [2.0, 3.0, 5.0, 6.0]
    assert n.storage() is t.storage()


def test_reshape_of_a_contiguous_tensor_is_a_view(be):
    t = t23(be)
    r = t.reshape((3, 2))
    assert [r.get_f32(i) for i in ([0, 1], [1, 0], [2, 1])] == [2.0, 3.0, 6.0]
    assert r.storage() is t.storage()


def test_contiguous_materializes_a_permuted_view(be):
    t = t23(be)
    tt = t.permute([1, 0])
    assert not tt.layout().is_contiguous()
    c = tt.contiguous()
    assert c.layout().is_contiguous() and c.storage() is not tt.storage()
    assert np.array_equal(c.to_host(), tt.to_host())
    assert t.contiguous().storage() is t.storage()  # no gratuitous copy


def test_view_errors_are_typed(be):
    t = t23(be)
    for bad in ([0, 0], [0]):
        with pytest.raises(ox.OxmeraError):
            t.permute(bad)
    with pytest.raises(ox.OxmeraError):
        t.narrow(1, 2, 2)
    with pytest.raises(ox.OxmeraError):
        t.narrow(2, 0, 1)
    with pytest.raises(ox.ShapeMismatch):
        t.reshape((4, 2))
    with pytest.raises(ox.ShapeMismatch):
        Tensor.from_host(np.ones(5, np.float32), (2, 3), DType.F32, be)


def test_permute_roundtrip_and_flip(be):
    rng = np.random.default_rng(2)
    for _ in range(20):
        dims = tuple(int(x) for x in rng.integers(1, 4, size=rng.integers(1, 4)))
        data = rng.uniform(-100, 100, ox.numel(dims)).astype(np.float32)
        t = Tensor.from_host(data, dims, DType.F32, be)
        rot = int(rng.integers(0, len(dims)))
        perm = [(i + rot) % len(dims) for i in range(len(dims))]
        inv = [0] * len(dims)
        for i, p in enumerate(perm):
            inv[p] = i
        assert np.array_equal(t.permute(perm).permute(inv).to_host(), data.reshape(dims))
        assert np.array_equal(t.permute(perm).to_host(), data.reshape(dims).transpose(perm))
        assert np.array_equal(t.flip(0).to_host(), data.reshape(dims)[::-1])


# ---- A5: exercises/a5-error-taxonomy/tests/spec.rs:11-81 ----
def test_device_kind_names():
    assert Device.cpu().kind_name() == "cpu"
    assert Device.metal(0).kind_name() == "metal"
    assert Device.cuda(1).kind_name() == "cuda"


def test_errors_are_self_describing():
    assert issubclass(ox.ShapeMismatch, Exception)
    e = ox.ShapeMismatch((2, 2), (2, 3), "matmul")
    assert "matmul" in str(e)
    e = ox.DeviceMismatch(Device.cpu(), Device.metal(0), "add")
    assert "add" in str(e) and "Cpu" in str(e) and "Metal" in str(e)
    with pytest.raises(ox.IndexOutOfBounds) as ei:
        Layout.contiguous((2, 3)).offset_of([0, 3])
    assert ei.value.index == [0, 3] and ei.value.shape == (2, 3) and "[0, 3]" in str(ei.value)
    with pytest.raises(ox.RankMismatch) as er:
        Layout.contiguous((2, 3)).offset_of([0])
    assert (er.value.index_rank, er.value.shape_rank) == (1, 2)
    with pytest.raises(ox.BroadcastIncompatible) as eb:
        ox.broadcast_shapes((2,), (3,))
    assert "2" in str(eb.value) and "3" in str(eb.value)


# ---- dispatch: crates/oxmera-runtime/tests/harness.rs:9-17 ----
def test_unregistered_device_is_a_typed_error(be):
    ox.unregister_all()
    with pytest.raises(ox.BackendUnavailable):
        ox.backend_for(Device.cuda(0))
    ox.register_backend(be)
    assert ox.backend_for(Device.cuda(0)) is be
    other = HostStandIn()
    ox.register_backend(other)  # replaces the previous registration
    assert ox.backend_for(Device.cuda(0)) is other
    ox.unregister_all()
