"""CPU: the arena layout of the one-kernel step's hand-over workspaces (dev_residency._ws_layout)."""
import pytest

from llamatov_b200 import dev_residency as dr


@pytest.mark.parametrize("sizes,cands", [([1792, 1792, 2304, 1792, 9728, 592], 12), ([64, 64, 96, 64, 128, 592], 3),
                                          ([57344, 57344, 2304, 57344, 311296, 592], 24)])
def test_candidate_windows_are_aligned_and_disjoint(sizes, cands):
    pitch, region, total = dr._ws_layout(sizes, cands)
    spans = []
    for i, n in enumerate(sizes):
        assert pitch[i] % 64 == 0 and (pitch[i] // 64) % 2 == 1        # an odd number of 256-byte units
        assert pitch[i] >= n                                           # windows of one vector do not overlap
        assert region[i] % 64 == 0                                     # 256-byte aligned (floats)
        for c in range(cands):
            spans.append((region[i] + c * pitch[i], region[i] + c * pitch[i] + n, i, c))
    spans.sort()
    for (a0, a1, *_), (b0, b1, *_) in zip(spans, spans[1:]):
        assert a1 <= b0
    assert spans[-1][1] <= total
