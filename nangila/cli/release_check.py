"""``python -m nangila.cli.release_check [--tag vX.Y.Z]``: consistency of a release.

Checks that ``release-manifest.toml``, the package's ``__version__`` and (when given) the git tag name
the same version, that every path of the stable and experimental surface exists, and that the
validation commands refer to files that are there. Exits non-zero with one line per problem.
The reference kept the same kind of manifest (nangila_v01/release-manifest.toml) and a checker behind
``make release-check``.
"""
from __future__ import annotations

import argparse
import glob
import os
import sys
import tomllib
from typing import List

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def check(tag: str | None = None, root: str = ROOT) -> List[str]:
    problems: List[str] = []
    path = os.path.join(root, "release-manifest.toml")
    if not os.path.exists(path):
        return [f"missing {path}"]
    with open(path, "rb") as fh:
        man = tomllib.load(fh)
    version = str(man.get("version", ""))
    from .. import __version__

    if version != __version__:
        problems.append(f"manifest version {version!r} != package version {__version__!r}")
    if man.get("git_tag") != f"v{version}":
        problems.append(f"manifest git_tag {man.get('git_tag')!r} != 'v{version}'")
    if tag is not None and tag != man.get("git_tag"):
        problems.append(f"tag {tag!r} != manifest git_tag {man.get('git_tag')!r}")
    scope = man.get("scope", {})
    for key in ("stable_surface", "experimental_surface"):
        for rel in scope.get(key, []):
            if not os.path.exists(os.path.join(root, rel)):
                problems.append(f"{key}: {rel} does not exist")
    overlap = set(scope.get("stable_surface", [])) & set(scope.get("experimental_surface", []))
    for rel in sorted(overlap):
        problems.append(f"{rel} is listed as both stable and experimental")
    for cmd in man.get("validation", {}).get("cpu", []) + man.get("validation", {}).get("gpu", []):
        for word in cmd.split():
            if word.endswith(".py") and not os.path.exists(os.path.join(root, word)):
                problems.append(f"validation command refers to a missing file: {word}")
    for pattern in man.get("artifacts", {}).get("native", []):
        if "*" not in pattern and not os.path.isdir(os.path.dirname(os.path.join(root, pattern))):
            problems.append(f"artifact directory missing for {pattern}")
    return problems


def built_artifacts(root: str = ROOT) -> List[str]:
    """Native artefacts of the manifest that are present in the tree (after ``python -m nangila._build``)."""
    with open(os.path.join(root, "release-manifest.toml"), "rb") as fh:
        man = tomllib.load(fh)
    out: List[str] = []
    for pattern in man.get("artifacts", {}).get("native", []):
        out += sorted(glob.glob(os.path.join(root, pattern)))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tag", default=None)
    args = ap.parse_args(argv)
    problems = check(args.tag)
    for p in problems:
        print("release-check: " + p)
    if not problems:
        print(f"release-check: ok ({len(built_artifacts())} native artefacts built in tree)")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
