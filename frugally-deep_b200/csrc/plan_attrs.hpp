// Indices into Op::a[] per operation kind, shared by the plan compiler and the executor.
#pragma once

namespace fdk {

enum ConvAttr : int {
    CONV_H = 0, CONV_W, CONV_C, CONV_HO, CONV_WO, CONV_KH, CONV_KW, CONV_SY, CONV_SX, CONV_DY, CONV_DX, CONV_PT, CONV_PL,
    CONV_DIRECT,      // 1x1 stride-1 unpadded: the input is the GEMM operand as it lies
    CONV_TRANSPOSED,  // gather from the undilated input (SY/SX are the dilation of the input)
    CONV_OFFY, CONV_OFFX, CONV_HD, CONV_WD,
    CONV_IMPLICIT,    // operand tiles are fetched by TMA straight from the NHWC input, no im2col buffer
    CONV_ROWWIN,      // few input channels: padded copy [HP][WP][CP] of the input, one k block per filter row
    CONV_RW_HP, CONV_RW_WP, CONV_RW_CP,
    CONV_PHASES,      // transposed: one implicit-GEMM launch per output phase with the layer's sub-filters (Layer::w_phases)
};
enum GemmAttr : int { GEMM_ROWS = 0 };
enum AffineAttr : int { AFF_OUTER = 0, AFF_NC, AFF_INNER, AFF_CONST };
enum NormAttr : int { NORM_ROWS = 0, NORM_N, NORM_RMS };
enum PoolAttr : int {
    POOL_PF = 0, POOL_PT, POOL_PL, POOL_MAX,
    POOL_FRAMED,                 // a preceding ZeroPadding layer was folded in: POOL_ZF.. hold its six pads
    POOL_ZF, POOL_ZB, POOL_ZT, POOL_ZBOT, POOL_ZL, POOL_ZR,
};
enum RnnAttr : int { RNN_T = 0, RNN_F, RNN_U };
enum MhaAttr : int { MHA_TQ = 0, MHA_TK };
enum BinOpCode : int { BINOP_ADD = 0, BINOP_SUB = 1, BINOP_MUL = 2, BINOP_MAX = 3, BINOP_MIN = 4 };

}  // namespace fdk
