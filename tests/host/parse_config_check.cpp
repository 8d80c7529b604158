// Host-side check of the drivers' grid-file parser (turbofno_b200/drivers/driver_config.h):
// prints, for the file given on the command line, every key with its values, one key per line
// ("key n v1 v2 ..."), in the order bs_list, dimX_list, DX_list, DY_list, N_list, K_list.
#include <cstdio>
#include <fstream>
#include <sstream>
#include "../../turbofno_b200/drivers/driver_config.h"

int main(int argc, char** argv) {
    if (argc != 2) { fprintf(stderr, "usage: %s <grid file>\n", argv[0]); return 2; }
    std::ifstream f(argv[1], std::ios::binary);
    if (!f) { fprintf(stderr, "cannot open %s\n", argv[1]); return 2; }
    std::stringstream ss;
    ss << f.rdbuf();
    auto grid = tfno_driver::parse_config(ss.str());
    for (const char* key : {"bs_list", "dimX_list", "DX_list", "DY_list", "N_list", "K_list"}) {
        auto it = grid.find(key);
        if (it == grid.end()) continue;
        printf("%s %zu", key, it->second.size());
        for (int v : it->second) printf(" %d", v);
        printf("\n");
    }
    return 0;
}
