#!/usr/bin/env bash
# Copy this checkout to a GPU host and build it there (no git, no rsync needed on the far side: tar over ssh).
#
#   server/deploy.sh user@gpu-host [remote-dir]        # default remote dir: ~/qw-b200
#
# Built libraries are not copied: the host libraries (g++) and the kernels (nvcc, sm_100a) are rebuilt in place on the
# target, which takes about half a minute.  Afterwards: ssh there and `server/ctl.sh start ...`.
set -euo pipefail

[ $# -ge 1 ] || { echo "usage: $0 user@host [remote-dir]" >&2; exit 2; }
target=$1
dir=${2:-qw-b200}
root=$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)

files() {
    # the tracked files of a git checkout; of a plain copy everything but built libraries and caches
    if git -C "$root" rev-parse --is-inside-work-tree >/dev/null 2>&1; then
        git -C "$root" ls-files -z | tar -C "$root" --null -T - -cf -
    else
        tar -C "$root" --exclude='*.so' --exclude=__pycache__ --exclude=.pytest_cache --exclude=build --exclude=build_checked -cf - .
    fi
}
files | ssh -o BatchMode=yes "$target" "mkdir -p $(printf '%q' "$dir") && tar -C $(printf '%q' "$dir") -xf - && cd $(printf '%q' "$dir") && python3 -m qwb200.build"
echo "deployed to $target:$dir"
