"""The build step's freshness rule: a source newer than the library means rebuild, and a build
dates the library at its start so that an edit made while the compiler ran is not lost."""

from __future__ import annotations

import os
import pathlib
import time

from paged_decode_attention_b200 import build as pbuild


def _fake_tree(tmp_path, monkeypatch):
    csrc = tmp_path / "pkg" / "csrc"
    csrc.mkdir(parents=True)
    (tmp_path / "include").mkdir()
    (tmp_path / "include" / "paged_decode.h").write_text("/* header */")
    for name in pbuild.SOURCES:
        (csrc / name).write_text("// source")
    lib = tmp_path / "pkg" / "lib.so"
    monkeypatch.setattr(pbuild, "PKG", tmp_path / "pkg")
    monkeypatch.setattr(pbuild, "CSRC", csrc)
    monkeypatch.setattr(pbuild, "LIB", lib)
    return csrc, lib


def test_needs_build_follows_modification_times(tmp_path, monkeypatch):
    csrc, lib = _fake_tree(tmp_path, monkeypatch)
    assert pbuild.needs_build()  # no library yet
    lib.write_bytes(b"")
    now = time.time()
    for f in list(csrc.iterdir()) + [tmp_path / "include" / "paged_decode.h"]:
        os.utime(f, (now - 100, now - 100))
    os.utime(lib, (now - 50, now - 50))
    assert not pbuild.needs_build()
    os.utime(csrc / pbuild.SOURCES[0], (now - 10, now - 10))  # edited after the library was made
    assert pbuild.needs_build()
    os.utime(csrc / pbuild.SOURCES[0], (now - 100, now - 100))
    os.utime(tmp_path / "include" / "paged_decode.h", (now, now))  # the header counts too
    assert pbuild.needs_build()


def test_build_dates_the_library_at_its_start(tmp_path, monkeypatch):
    csrc, lib = _fake_tree(tmp_path, monkeypatch)

    class FakeProc:
        returncode = 0

        def communicate(self):
            return "", None

    def fake_popen(cmd, **kw):  # "compiling": a source is edited while the compiler runs
        time.sleep(0.05)
        (csrc / pbuild.SOURCES[0]).write_text("// edited during the build")
        return FakeProc()

    def fake_run(cmd, check):  # "linking": to the output the command names, never straight to the library
        out = pathlib.Path(cmd[cmd.index("-o") + 1])
        assert out != lib, "the link must not write the library in place"
        out.write_bytes(b"linked")

    monkeypatch.setattr(pbuild, "_nvcc", lambda: "nvcc")
    monkeypatch.setattr(pbuild.subprocess, "Popen", fake_popen)
    monkeypatch.setattr(pbuild.subprocess, "run", fake_run)
    pbuild.build(force=True)
    assert lib.exists() and lib.read_bytes() == b"linked"
    assert [p.name for p in lib.parent.iterdir() if p.name.startswith(lib.name) and p != lib] == []
    assert pbuild.needs_build(), "the edit made during the build must trigger the next build"
