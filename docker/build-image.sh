#!/usr/bin/env bash
# Build the engine's image from this checkout, here or on a remote docker host.
#
#   docker/build-image.sh                      # local docker
#   docker/build-image.sh user@gpu-host        # the tree goes over ssh as a tar stream; nothing is cloned there
#   docker/build-image.sh user@gpu-host tag
#
# The image is tagged qw-b200:<short commit> (or the tag given) and qw-b200:latest.  Only tracked files go into the build
# context (no built libraries, caches or history); the kernels are compiled inside the image.
set -euo pipefail

root=$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)
where=${1:-local}
rev=$(git -C "$root" rev-parse --short HEAD 2>/dev/null || echo dev)
tag=${2:-qw-b200:$rev}

context() {
    # the tracked files of a git checkout; of a plain copy everything but built libraries and caches
    if git -C "$root" rev-parse --is-inside-work-tree >/dev/null 2>&1; then
        git -C "$root" ls-files -z | tar -C "$root" --null -T - -cf -
    else
        tar -C "$root" --exclude='*.so' --exclude=__pycache__ --exclude=.pytest_cache --exclude=build --exclude=build_checked -cf - .
    fi
}
build=(docker build -t "$tag" -t qw-b200:latest -f docker/Dockerfile -)

if [ "$where" = local ]; then
    context | "${build[@]}"
else
    context | ssh "$where" "$(printf '%q ' "${build[@]}")"
fi
echo "built $tag on $where"
