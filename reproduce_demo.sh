#!/usr/bin/env bash
# Three short synthetic runs (dense, STAC-R, Turbo-fast) through the generic trainer; extra arguments are passed on.
set -euo pipefail
cd -- "$(dirname -- "${BASH_SOURCE[0]}")"
device="${STACR_DEVICE:-cpu}"
for method in baseline stacr turbofast; do
  python -m stacr train --config synthetic_stacr --device "$device" --set "method=$method" --output "outputs/demo/$method.csv" "$@"
done
python -m scripts.aggregate_results --input outputs/demo --output outputs/demo/demo_results.csv
