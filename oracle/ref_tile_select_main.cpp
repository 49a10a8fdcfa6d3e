// Driver around the reference's own select_optimal_tile (wmma_tile_selection.hpp:30-66),
// compiled from the reference tree by oracle/Makefile. Reads "M N K" triples from stdin and
// prints "M N K config" per line. Used to pin oracle/tile_plan.py and to generate
// tests/golden/tile_selection.json.
#include <cstdio>

#include "wmma_tile_selection.hpp"

int main() {
    int M, N, K;
    while (std::scanf("%d %d %d", &M, &N, &K) == 3)
        std::printf("%d %d %d %d\n", M, N, K, static_cast<int>(select_optimal_tile(M, N, K)));
    return 0;
}
