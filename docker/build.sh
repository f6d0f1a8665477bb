#!/bin/bash
# Build the container image of this repository from its root directory.
#   docker/build.sh [tag] [base image]
set -euo pipefail
tag="${1:-makani-b200:latest}"
base="${2:-nvcr.io/nvidia/pytorch:25.03-py3}"
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
docker build --network host -t "${tag}" --build-arg BASE="${base}" -f "${here}/Dockerfile" "${here}/.."
