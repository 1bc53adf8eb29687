"""The arithmetic by which the large-M kernel's persistent CTAs share a launch (``nnfusion_b200/csrc/dq_gemm_tcgen05.cu``:
``WorkList``, ``cta_of_unit``, ``slot_of``), restated in Python and checked for the properties the kernel relies on:
the shares partition the units, every share splits into segments that lie inside one tile, a share has at most two
tiles that it does not compute alone (its first and its last: one workspace slot each), and every CTA that the
formula names as a contributor to a shared tile really has a segment of that tile."""
import itertools

import pytest


def shares(tiles, cpt, G):
    U = tiles * cpt
    return [(c * U // G, (c + 1) * U // G) for c in range(G)]


def segments(u, u_end, cpt):
    out = []
    while u < u_end:
        tile, c0 = divmod(u, cpt)
        c1 = min(cpt, c0 + (u_end - u))
        out.append((tile, c0, c1))
        u += c1 - c0
    return out


def cta_of_unit(u, U, G):
    return ((u + 1) * G + U - 1) // U - 1


def slot_of(c, t, U, G, cpt):
    first_tile = (c * U // G) // cpt
    return 2 * c + (0 if t == first_tile else 1)


@pytest.mark.parametrize("tiles,cpt,G", [
    (86, 16, 148), (172, 16, 148), (344, 16, 148), (1376, 16, 148), (8, 16, 128), (32, 8, 148), (3584, 32, 148),
    (1, 1, 1), (1, 5, 5), (3, 2, 6), (7, 3, 4), (149, 1, 148), (148, 43, 148), (5, 172, 148), (1000, 7, 132)])
def test_shares_and_slots(tiles, cpt, G):
    U = tiles * cpt
    assert G <= U                                     # the host never launches more CTAs than units
    sh = shares(tiles, cpt, G)
    assert sh[0][0] == 0 and sh[-1][1] == U
    assert all(a[1] == b[0] for a, b in zip(sh, sh[1:]))        # a partition, in order
    assert all(e > b for b, e in sh)                            # nobody is idle
    used_slots = set()
    contributors = {}                                           # tile -> CTAs with a partial segment of it
    for c, (b, e) in enumerate(sh):
        segs = segments(b, e, cpt)
        assert sum(c1 - c0 for _, c0, c1 in segs) == e - b
        partial = [(i, t) for i, (t, c0, c1) in enumerate(segs) if not (c0 == 0 and c1 == cpt)]
        assert all(i in (0, len(segs) - 1) for i, _ in partial)  # only the first and the last can be shared
        for _, t in partial:
            s = slot_of(c, t, U, G, cpt)
            assert s not in used_slots and 0 <= s < 2 * G
            used_slots.add(s)
            contributors.setdefault(t, []).append(c)
        for u in (b, e - 1, (b + e) // 2):
            assert cta_of_unit(u, U, G) == c
    for t, ctas in contributors.items():
        first, last = cta_of_unit(t * cpt, U, G), cta_of_unit((t + 1) * cpt - 1, U, G)
        assert ctas == list(range(first, last + 1))             # consecutive CTAs, each with its piece, K order
        assert len(ctas) >= 2                                   # a tile with one contributor is computed whole


def test_whole_tile_mode_cuts_at_tile_boundaries():
    for tiles, cpt, G in itertools.product((1, 5, 86, 128, 148), (1, 4, 16), (1, 86, 148)):
        if G > tiles:
            continue
        cuts = [c * tiles // G * cpt for c in range(G + 1)]
        assert cuts[0] == 0 and cuts[-1] == tiles * cpt
        for b, e in zip(cuts, cuts[1:]):
            assert e > b and all(c0 == 0 and c1 == cpt for _, c0, c1 in segments(b, e, cpt))
