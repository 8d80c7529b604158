// Problem-size grid files of the drivers: "<key> = v1 v2 ..." per line, '#' comments and blank
// lines skipped, keys bs_list, dimX_list | DX_list, DY_list, N_list, K_list
// (format of benchmark_config/problem_size_{1d,2d}.txt in the reference; parsed there by
// parse_line, utils/utils.cu:14-22, and the loop at
// fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:84-97).
#pragma once
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

namespace tfno_driver {

// Values of one line; tokens after "<key> =" that are not integers end the list.
inline std::vector<int> parse_values(const std::string& line) {
    std::vector<int> out;
    std::istringstream in(line);
    std::string key, eq;
    in >> key >> eq;
    for (int v; in >> v;) out.push_back(v);
    return out;
}

inline std::unordered_map<std::string, std::vector<int>> parse_config(const std::string& text) {
    std::unordered_map<std::string, std::vector<int>> grid;
    std::istringstream in(text);
    std::string line;
    while (std::getline(in, line)) {
        if (!line.empty() && line.back() == '\r') line.pop_back();
        if (line.empty() || line[0] == '#') continue;
        std::istringstream first(line);
        std::string key;
        first >> key;
        if (key.empty()) continue;
        grid[key] = parse_values(line);
    }
    return grid;
}

}  // namespace tfno_driver
