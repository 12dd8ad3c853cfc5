#!/usr/bin/env bash
# The four GPT-2-medium quality protocols (dense, checkpointing, STAC-R, Turbo-fast). STACR_STEPS shortens them.
set -euo pipefail
cd -- "$(dirname -- "${BASH_SOURCE[0]}")"
extra=()
if [[ -n "${STACR_STEPS:-}" ]]; then extra+=(--steps "$STACR_STEPS"); fi
for arm in baseline checkpoint full turbo; do
  python -m stacr reproduce run "gpt2-medium-quality-$arm" "${extra[@]}" "$@"
done
