# Tylo on libtylo_b200: the exported API of Tylo.jl with every kernel launch replaced by a ccall
# into the sm_100a library (include/tylo_b200.h).  No cuTile.jl, no kernel code in Julia, no CPU
# fallback: a request the library has no kernel for throws.
#
# NOTE: this package was written against the frozen C header and could not be executed where the
# library is built and tested (no Julia there).  The three spellings that depend on the CUDA.jl /
# CUDACore version in use are isolated in `src/lib.jl` (`devptr`, `current_stream`, `is_dense`).
module Tylo

using CUDACore
using CUDACore: CuArray
using Adapt: Adapt, adapt

include("lib.jl")
include("buffers.jl")
include("attention/mods.jl")
include("attention/pair.jl")
include("attention/flex.jl")
include("attention/attention.jl")
include("attention/decode.jl")
include("softmax/softmax.jl")
include("norm/rms_norm.jl")
include("norm/layer_norm.jl")

end
