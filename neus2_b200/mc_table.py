"""A marching-cubes case table generated from first principles, for callers that do not bring their own.

Numbering follows the reference's kernels (src/marching_cubes.cu:260-275): corners 0-3 run around the z = 0 face
(0,0,0) (1,0,0) (1,1,0) (0,1,0), corners 4-7 the same at z = 1; edges 0-3 and 4-7 follow the two rings, edges 8-11 go
up from corners 0-3.  For each of the 256 corner patterns the crossed edges are linked face by face (on a face with four
crossings each 'inside' corner is cut off on its own, a rule that only looks at the face, so neighbouring cubes agree
and the mesh is watertight), the links close into loops, each loop is triangulated without diagonals that lie in a cube face and
oriented with its normal towards the corners whose value is above the threshold.  The triangulation is valid but not necessarily the same as
another table's: pass the reference's own table to reproduce its topology."""
import numpy as np

CORNERS = np.array([(0, 0, 0), (1, 0, 0), (1, 1, 0), (0, 1, 0), (0, 0, 1), (1, 0, 1), (1, 1, 1), (0, 1, 1)], np.float64)
EDGES = [(0, 1), (1, 2), (2, 3), (3, 0), (4, 5), (5, 6), (6, 7), (7, 4), (0, 4), (1, 5), (2, 6), (3, 7)]
# faces as cyclic corner quadruples
FACES = [(0, 1, 2, 3), (4, 5, 6, 7), (0, 1, 5, 4), (1, 2, 6, 5), (2, 3, 7, 6), (3, 0, 4, 7)]
_EDGE_OF = {frozenset(e): i for i, e in enumerate(EDGES)}
_table = None


def _links(mask):
    """Directed links {from edge: to edge}: on every face the contour runs with the 'above' corners on its left as seen from
    outside the cube (triangle normals then point towards the corners above the threshold, the reference table's winding), so the links of a pattern chain into oriented loops and neighbouring cubes traverse a shared face's
    segment in opposite directions (a consistently oriented mesh)."""
    above = [(mask >> i) & 1 for i in range(8)]
    mid = [(CORNERS[a] + CORNERS[b]) / 2 for a, b in EDGES]
    nxt = {}
    for f in FACES:
        outward = CORNERS[list(f)].mean(0) - 0.5
        crossed = []  # (edge id, corner of the face that is 'above' on that edge)
        for k in range(4):
            a, b = f[k], f[(k + 1) % 4]
            if above[a] != above[b]:
                crossed.append((_EDGE_OF[frozenset((a, b))], a if above[a] else b))
        pairs = []
        if len(crossed) == 2:
            pairs.append((crossed[0][0], crossed[1][0], crossed[0][1]))
        elif len(crossed) == 4:  # two 'above' corners on a diagonal: cut each off on its own
            by_corner = {}
            for e, c in crossed:
                by_corner.setdefault(c, []).append(e)
            for c, es in by_corner.items():
                pairs.append((es[0], es[1], c))
        for e0, e1, c in pairs:
            if np.dot(np.cross(mid[e1] - mid[e0], CORNERS[c] - mid[e0]), outward) < 0:
                e0, e1 = e1, e0
            assert e0 not in nxt
            nxt[e0] = e1
    return nxt


def _on_one_face(e0, e1):
    c = set(EDGES[e0]) | set(EDGES[e1])
    return any(c <= set(f) for f in FACES)


def _triangulate(loop):
    """Triangles of a loop with no inner diagonal lying in a face of the cube: such a diagonal would coincide with the
    neighbouring cube's and make a non-manifold edge.  First admissible triangulation in a fixed enumeration order."""
    def rec(poly):
        if len(poly) == 3:
            return [list(poly)]
        a, b = poly[0], poly[-1]  # the side (b, a) is a polygon side or an already accepted diagonal
        for k in range(1, len(poly) - 1):
            if (k > 1 and _on_one_face(a, poly[k])) or (k < len(poly) - 2 and _on_one_face(poly[k], b)):
                continue
            left = rec(poly[:k + 1]) if k > 1 else []
            right = rec(poly[k:]) if k < len(poly) - 2 else []
            if left is None or right is None:
                continue
            return left + [[a, poly[k], b]] + right
        return None
    tris = rec(list(loop))
    assert tris is not None, loop
    return [e for t in tris for e in t]


def make_table():
    global _table
    if _table is not None:
        return _table
    table = np.full((256, 16), -1, np.int8)
    for mask in range(1, 255):
        nxt = _links(mask)
        seen, tris = set(), []
        for start in sorted(nxt):
            if start in seen:
                continue
            loop, cur = [], start
            while cur not in seen:
                seen.add(cur)
                loop.append(cur)
                cur = nxt[cur]
            assert cur == start and len(loop) >= 3
            tris += _triangulate(loop)
        assert len(tris) <= 15, (mask, tris)
        table[mask, :len(tris)] = tris
    _table = table
    return table
