"""Writes tests/golden/reference_conv_fwd_1d_3d.json.

The expected values are the golden vectors of the reference's host test of its CPU convolution for the 1-D and 3-D
cases (test/reference_conv_fwd/reference_conv_fwd.cpp: Conv1DNWC, Conv1DNWCStridesDilationsPadding, Conv3DNCDHW,
Conv3DNCDHWStridesDilations).  This script reads the `ref_data` initialisers of those tests from the reference
checkout (only here, when the fixture is made; the tests use the committed JSON), re-derives every value with exact
integer arithmetic (no oracle code involved) and stores both:
  1-D: NWC input filled 0, 1, 2, ... in memory order (FillMonotonicSeq, fill.hpp:65-81), weights 0.5;
  3-D: NCDHW input filled 0, 0.1, 0.2, ... in memory order, weights 0.5, output listed in NKDHW order.
The reference's own check uses check_err's float tolerance (its numbers carry float32 rounding: 410.40002), so the
re-derivation is compared with rtol 1e-5.
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_TEST = os.path.join("test", "reference_conv_fwd", "reference_conv_fwd.cpp")  # inside the reference checkout


def ref_data_of(text, test_name):
    body = text[text.index("TEST(ReferenceConvolutionFWD, %s)" % test_name):]
    init = body[body.index("ref_data{") + len("ref_data{"):]
    init = init[:init.index("}")]
    return [float(t) for t in re.findall(r"-?\d+\.?\d*(?:e-?\d+)?", init)]


def derive(nd, N, K, C, in_sp, filt, stride, dil, pad, channel_first, step_num, step_den):
    """Integer sum of input indices under each output's window; value = sum * step * 0.5.
    Returns the output as a flat list in (N, K, spatial...) order (channel_first) or (N, spatial..., K)."""
    sp3 = [1] * (3 - nd) + list(in_sp)
    f3 = [1] * (3 - nd) + list(filt)
    s3 = [1] * (3 - nd) + list(stride)
    d3 = [1] * (3 - nd) + list(dil)
    p3 = [0] * (3 - nd) + list(pad)
    o3 = [(sp3[i] + 2 * p3[i] - ((f3[i] - 1) * d3[i] + 1)) // s3[i] + 1 for i in range(3)]

    def in_index(n, c, d, h, w):
        if channel_first:
            return (((n * C + c) * sp3[0] + d) * sp3[1] + h) * sp3[2] + w
        return (((n * sp3[0] + d) * sp3[1] + h) * sp3[2] + w) * C + c

    vals = {}
    for n in range(N):
        for k in range(K):
            for od in range(o3[0]):
                for oh in range(o3[1]):
                    for ow in range(o3[2]):
                        acc = 0
                        for c in range(C):
                            for z in range(f3[0]):
                                for y in range(f3[1]):
                                    for x in range(f3[2]):
                                        d, h, w = (od * s3[0] + z * d3[0] - p3[0], oh * s3[1] + y * d3[1] - p3[1],
                                                   ow * s3[2] + x * d3[2] - p3[2])
                                        if 0 <= d < sp3[0] and 0 <= h < sp3[1] and 0 <= w < sp3[2]:
                                            acc += in_index(n, c, d, h, w)
                        vals[(n, k, od, oh, ow)] = acc * step_num / (2.0 * step_den)
    keys = sorted(vals) if channel_first else sorted(vals, key=lambda t: (t[0], t[2], t[3], t[4], t[1]))
    return o3[3 - nd:], [vals[k] for k in keys]


CASES = [
    ("Conv1DNWC", dict(nd=1, N=1, K=1, C=2, in_sp=[6], filt=[3], stride=[1], dil=[1], pad=[0]), False, (1, 1)),
    ("Conv1DNWCStridesDilationsPadding",
     dict(nd=1, N=1, K=2, C=2, in_sp=[12], filt=[3], stride=[2], dil=[2], pad=[1]), False, (1, 1)),
    ("Conv3DNCDHW", dict(nd=3, N=1, K=1, C=2, in_sp=[6, 6, 6], filt=[3, 3, 3], stride=[1, 1, 1], dil=[1, 1, 1],
                         pad=[0, 0, 0]), True, (1, 10)),
    ("Conv3DNCDHWStridesDilations",
     dict(nd=3, N=1, K=2, C=2, in_sp=[12, 12, 12], filt=[3, 3, 3], stride=[3, 3, 3], dil=[1, 1, 1], pad=[0, 0, 0]),
     True, (1, 10)),
]


def main():
    if len(sys.argv) != 2 or not os.path.exists(os.path.join(sys.argv[1], REF_TEST)):
        sys.exit("usage: make_convnd_golden.py <root of the reference checkout>   (needs " + REF_TEST + ")")
    text = open(os.path.join(sys.argv[1], REF_TEST)).read()
    cases = []
    for name, geom, channel_first, (num, den) in CASES:
        expected = ref_data_of(text, name)
        out_sp, derived = derive(channel_first=channel_first, step_num=num, step_den=den, **geom)
        assert len(derived) == len(expected), (name, len(derived), len(expected))
        for a, b in zip(derived, expected):
            assert abs(a - b) <= 1e-5 * abs(b) + 1e-6, (name, a, b)
        cases.append(dict(name=name, geometry=geom, output_spatial=out_sp,
                          input_fill="memory-order monotonic sequence, step %d/%d, %s layout" %
                                     (num, den, "NCDHW" if channel_first else "NWC"),
                          input_step=num / den, weights=0.5,
                          output_order="N,K,spatial" if channel_first else "N,spatial,K",
                          expected=expected, derived=derived))
    with open(os.path.join(HERE, "reference_conv_fwd_1d_3d.json"), "w") as f:
        json.dump(dict(source="test/reference_conv_fwd/reference_conv_fwd.cpp (Conv1DNWC*, Conv3DNCDHW*)",
                       cases=cases), f, indent=1)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
