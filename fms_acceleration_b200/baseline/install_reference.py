"""Place the reference project under ``baseline/_ref`` of the repository checkout.

    python -m fms_acceleration_b200.baseline.install_reference <path-to-reference-checkout>

First the offline ``pip install --target`` that a packaged project would need is tried (the outcome is written to
``baseline/_ref/INSTALL_LOG.txt``); the reference is a monorepo of seven packages without a top-level build file and
with build backends / dependencies that are not available offline, so the fallback, a plain copy of every plugin's
``src/<package>`` directory, is what normally ends up there.  Nothing is modified: the baseline backend loads single
kernel files from that copy by path (see ``backend.py``), and ``bench.py --impl reference`` reports the import error it
hits when it tries the reference's own public API."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None) -> int:
    argv = argv if argv is not None else sys.argv[1:]
    if not argv:
        print(__doc__)
        return 2
    src = os.path.abspath(argv[0])
    dst = os.path.join(REPO, "baseline", "_ref")
    os.makedirs(dst, exist_ok=True)
    log = []
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links", "/opt/wheelhouse",
           "--target", dst, src]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log.append("$ " + " ".join(cmd))
    log.append(f"exit code {res.returncode}")
    log.append((res.stdout + res.stderr).strip()[-2000:])
    copied = []
    plugins = os.path.join(src, "plugins")
    if os.path.isdir(plugins):
        for plug in sorted(os.listdir(plugins)):
            pkg_root = os.path.join(plugins, plug, "src")
            if not os.path.isdir(pkg_root):
                continue
            for pkg in sorted(os.listdir(pkg_root)):
                s, d = os.path.join(pkg_root, pkg), os.path.join(dst, pkg)
                if os.path.isdir(s) and not os.path.exists(d):
                    shutil.copytree(s, d, ignore=shutil.ignore_patterns("__pycache__"))
                    copied.append(pkg)
    log.append("plain copy of: " + (", ".join(copied) if copied else "(nothing new)"))
    with open(os.path.join(dst, "INSTALL_LOG.txt"), "w", encoding="utf-8") as fh:
        fh.write("\n".join(log) + "\n")
    print("\n".join(log))
    return 0


if __name__ == "__main__":
    sys.exit(main())
