"""The reference's WMMA example scripts (examples/wmma/*.jl of CUDAnative.jl), statement for statement,
against this package."""
