"""Host-side handling of the C ABI's status codes and of the device status word (no GPU needed)."""
import pytest

import bioemu2_b200._lib as L


class _FakeLib:
    def __init__(self, msg):
        self._msg = msg

    def b200_last_error(self):
        return self._msg


@pytest.mark.parametrize("code,exc", [
    (L.ERR_INVALID_ARGUMENT, ValueError),
    (L.ERR_WORKSPACE, ValueError),
    (L.ERR_CUDA, RuntimeError),
    (L.ERR_UNSUPPORTED_DEVICE, RuntimeError),
    (L.ERR_DEVICE_WAIT, L.DeviceWaitError),
])
def test_status_code_becomes_the_matching_exception(monkeypatch, code, exc):
    monkeypatch.setattr(L, "lib", _FakeLib(b"what went wrong"))
    with pytest.raises(exc, match="what went wrong"):
        L.check(code)


def test_ok_raises_nothing(monkeypatch):
    monkeypatch.setattr(L, "lib", _FakeLib(b""))
    L.check(L.OK)


def test_device_wait_is_a_runtime_error():
    assert issubclass(L.DeviceWaitError, RuntimeError)


def test_status_word_decoding():
    assert L.decode_status(0) == "ok"
    word = 1 | (67 << 8)  # kind 1 (wait ran out), site 67
    text = L.decode_status(word)
    assert "wait site 67" in text and "bounded wait ran out" in text and hex(word) in text
    assert "unknown kind 9" in L.decode_status(9 | (3 << 8))


def test_header_and_binding_agree_on_every_symbol():
    """Every function include/b200pair.h declares is bound, with the declared number of arguments, and exported."""
    import os
    import re

    header = open(os.path.join(os.path.dirname(L.HERE), "include", "b200pair.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    decls = re.findall(r"\b(b200_\w+)\s*\(([^;{]*?)\)\s*;", header)
    assert len(decls) >= 30
    for name, args in decls:
        assert name in L.SIGNATURES, f"{name} is declared but not bound"
        n_args = 0 if args.strip() in ("", "void") else args.count(",") + 1
        assert len(L.SIGNATURES[name][1]) == n_args, f"{name}: header has {n_args} arguments"
        assert hasattr(L.lib, name)
    assert {n for n, _ in decls} == set(L.SIGNATURES), "binding has functions the header does not declare"
