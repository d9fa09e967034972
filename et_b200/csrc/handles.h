// Opaque C-ABI handle types shared by the translation units that create and consume them.
#pragma once
#include "tile_gemm.h"

struct et_tile_weight {
    et::TileWeight* w;
};
