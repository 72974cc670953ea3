"""Two processes that find the library stale at the same moment (two ranks of one job sharing the tree) must not
compile twice nor leave a half-written file for the other to load.  A stand-in ``nvcc`` (a shell script that logs and
sleeps) replaces the compiler, and the package's paths are pointed at a scratch tree, so nothing real is built."""
from __future__ import annotations

import os
import stat
import subprocess
import sys
import textwrap
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent(
    """
    import sys
    from pathlib import Path
    sys.path.insert(0, {repo!r})
    from baybridge_b200.backend import native
    root = Path({root!r})
    native.PACKAGE_DIR = root
    native.CSRC_DIR = root / "csrc"
    native.LIBRARY_PATH = root / "libbb200.so"
    native.STAMP_PATH = root / "libbb200.stamp"
    native.build_library()
    assert native.library_is_current()
    print(native.LIBRARY_PATH.read_text().strip())
    """
)

FAKE_NVCC = textwrap.dedent(
    """\
    #!/bin/sh
    # stand-in compiler: the argument after -o is the output; record the call, take a while, write the output whole
    out=""
    prev=""
    for a in "$@"; do
      if [ "$prev" = "-o" ]; then out="$a"; fi
      prev="$a"
    done
    echo "$out" >> "$FAKE_NVCC_LOG"
    printf 'partial' > "$out"
    sleep 0.5
    printf 'complete\\n' > "$out"
    """
)


def test_concurrent_builders_compile_once_and_never_expose_a_partial_library(tmp_path):
    root = tmp_path / "pkg"
    (root / "csrc").mkdir(parents=True)
    (root / "csrc" / "one.cu").write_text("// a\n")
    (root / "csrc" / "two.cu").write_text("// b\n")
    (tmp_path / "include").mkdir()
    (tmp_path / "include" / "bb200.h").write_text("// header\n")
    bin_dir = tmp_path / "bin"
    bin_dir.mkdir()
    fake = bin_dir / "nvcc"
    fake.write_text(FAKE_NVCC)
    fake.chmod(fake.stat().st_mode | stat.S_IXUSR)
    log = tmp_path / "nvcc.log"
    env = dict(os.environ, PATH=f"{bin_dir}:{os.environ['PATH']}", FAKE_NVCC_LOG=str(log))
    code = CHILD.format(repo=str(REPO), root=str(root))
    children = [subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
                for _ in range(3)]
    results = [child.communicate(timeout=120) for child in children]
    for child, (out, err) in zip(children, results):
        assert child.returncode == 0, err
        assert out.strip() == "complete"
    calls = log.read_text().split()
    # two objects and one link, once: the processes that waited on the lock found the library current
    assert len(calls) == 3, calls
    assert sum(name.endswith(".o") for name in calls) == 2
    assert (root / "libbb200.so").read_text() == "complete\n"
    assert not list((root / "build").glob("libbb200.*.so"))
