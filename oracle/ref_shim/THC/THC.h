// TEST INFRASTRUCTURE.  Empty stand-in for the header of the same name that PyTorch removed after 1.x.
// The reference's operator sources (src/ops/dgl_primitives/bcast.h:8, spmm.cu:10, sddmm.cu:8) include it
// but use nothing that it declared; this file lets them compile unmodified where they lie.
#pragma once
