#!/bin/bash
# Builds the shared library and the ten TurboFNO_{1D,2D}_{A..E} executables in one go and writes
# envpath.sh, which puts them on PATH -- the job of the reference's install.sh (install.sh:13-24
# loops over the variant directories, :59-66 writes envpath.sh with one PATH export per variant).
# Here the ten programs come from one source and land in one directory, so envpath.sh has one line.
#
#   ./install.sh          build everything that is out of date
#   ./install.sh clean    remove the built library and executables (install.sh:27-41 in the reference)
set -e
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(dirname "$HERE")"
if [ "$1" = "clean" ]; then
    rm -rf "$HERE/bin" "$HERE/libturbofno_b200.so" "$HERE/libturbofno_b200.so.srchash" "$HERE/envpath.sh"
    echo "cleaned"
    exit 0
fi
cd "$ROOT"
python -m turbofno_b200.build --drivers
echo "export PATH=\"$HERE/bin:\$PATH\"" > "$HERE/envpath.sh"
echo "export LD_LIBRARY_PATH=\"$HERE:\$LD_LIBRARY_PATH\"" >> "$HERE/envpath.sh"
echo "wrote $HERE/envpath.sh  (source it to put TurboFNO_1D_A ... TurboFNO_2D_E on PATH)"
