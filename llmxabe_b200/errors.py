"""Status codes of the C ABI as exceptions named after the reference's error
variants (crates/xabe-cuda/src/kernels/moe.rs:4602-4637 `MoeError`,
crates/xabe-engine/src/block/moe.rs:493-547 `MoeBlockError`)."""


class MoeError(RuntimeError):
    code = -1


class UnsupportedGeometry(MoeError):
    code = 1


class RaggedWeights(MoeError):
    code = 2


class WrongElementCount(MoeError):
    code = 3


class TooManyTokens(MoeError):
    code = 4


class SharedOnlyBuffers(MoeError):
    code = 5


class Driver(MoeError):
    code = 6


class BufferLength(MoeError):
    code = 7


class UnsupportedExpertType(MoeError):
    code = 8


class UnsupportedDenseType(MoeError):
    code = 9


class InvalidArgument(MoeError):
    code = 10


class DeviceStatus(MoeError):
    code = 11


_BY_CODE = {c.code: c for c in (UnsupportedGeometry, RaggedWeights, WrongElementCount, TooManyTokens,
                                SharedOnlyBuffers, Driver, BufferLength, UnsupportedExpertType,
                                UnsupportedDenseType, InvalidArgument, DeviceStatus)}


def check(code: int, message: bytes | str | None) -> None:
    if code == 0:
        return
    if isinstance(message, bytes):
        message = message.decode("utf-8", "replace")
    raise _BY_CODE.get(code, MoeError)(message or f"status {code}")
