"""Writes tests/golden/reference_conv_fwd_2d.json.

The expected values are the golden vectors the reference's own host test holds for its CPU
convolution (test/reference_conv_fwd/reference_conv_fwd.cpp:94-154).  That test fills the NHWC
input with 0, 1, 2, ... in memory order (FillMonotonicSeq, library/include/ck/library/utility/
fill.hpp:65-81) and every weight with 0.5 (FillConstant, fill.hpp:83-93), so each value below can
be re-derived by hand: e.g. case 1, output (0,0) = 0.5 * sum over the 3x3x2 window starting at
pixel (0,0) = 0.5 * 261 = 130.5.  This script re-derives them with plain integer arithmetic
(no oracle code involved) and stores them next to the expectation stated in the reference test,
so that the fixture is checked twice: re-derivation == reference's numbers, and oracle == fixture.
"""
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))

# numbers as they appear in the reference test (file:line in the docstring above)
CASE1_EXPECTED = [130.5, 148.5, 166.5, 184.5, 238.5, 256.5, 274.5, 292.5,
                  346.5, 364.5, 382.5, 400.5, 454.5, 472.5, 490.5, 508.5]
CASE2_EXPECTED = [
    210., 210., 327., 327., 351., 351., 375., 375., 399., 399.,
    459., 459., 706.5, 706.5, 742.5, 742.5, 778.5, 778.5, 814.5, 814.5,
    747., 747., 1138.5, 1138.5, 1174.5, 1174.5, 1210.5, 1210.5, 1246.5, 1246.5,
    1035., 1035., 1570.5, 1570.5, 1606.5, 1606.5, 1642.5, 1642.5, 1678.5, 1678.5,
    1323., 1323., 2002.5, 2002.5, 2038.5, 2038.5, 2074.5, 2074.5, 2110.5, 2110.5]


def derive(N, K, C, Hi, Wi, Y, X, s, d, p):
    Ho = (Hi + 2 * p - ((Y - 1) * d + 1)) // s + 1
    Wo = (Wi + 2 * p - ((X - 1) * d + 1)) // s + 1
    out = []
    for n in range(N):
        for ho in range(Ho):
            for wo in range(Wo):
                for k in range(K):
                    acc = 0
                    for y in range(Y):
                        for x in range(X):
                            hi, wi = ho * s + y * d - p, wo * s + x * d - p
                            if 0 <= hi < Hi and 0 <= wi < Wi:
                                for c in range(C):
                                    acc += ((n * Hi + hi) * Wi + wi) * C + c
                    out.append(acc * 0.5)
    return (N, Ho, Wo, K), out


def main():
    cases = []
    for name, geom, expected in [
        ("Conv2DNHWC", dict(N=1, K=1, C=2, Hi=6, Wi=6, Y=3, X=3, s=1, d=1, p=0), CASE1_EXPECTED),
        ("Conv2DNHWCStridesDilationsPadding", dict(N=1, K=2, C=2, Hi=12, Wi=12, Y=3, X=3, s=2, d=2, p=1),
         CASE2_EXPECTED),
    ]:
        shape, derived = derive(**geom)
        assert derived == expected, (name, derived, expected)
        cases.append(dict(name=name, geometry=geom, output_shape_nhwk=list(shape), expected=expected,
                          input="memory-order monotonic sequence 0,1,2,...", weights="constant 0.5"))
    out_len = [  # test/conv_util/conv_util.cpp:43-79: (Hi, Y, stride, dilation, lpad, rpad) -> Ho
        dict(args=[71, 3, 2, 1, 1, 1], expected=36),
        dict(args=[71, 3, 1, 1, 1, 1], expected=71),
        dict(args=[71, 3, 2, 1, 2, 2], expected=37),
        dict(args=[71, 3, 2, 2, 2, 2], expected=36),
        dict(args=[71, 3, 3, 2, 1, 1], expected=23),
    ]
    with open(os.path.join(HERE, "reference_conv_fwd_2d.json"), "w") as f:
        json.dump(dict(source="test/reference_conv_fwd/reference_conv_fwd.cpp:94-154; "
                              "test/conv_util/conv_util.cpp:43-79",
                       conv_cases=cases, output_length_cases=out_len), f, indent=1)


if __name__ == "__main__":
    main()
