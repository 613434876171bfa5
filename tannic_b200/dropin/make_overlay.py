"""Generates the "fused by default" header overlay for the reference's front-end.

    python make_overlay.py <reference source tree> <output directory>

The reference evaluates an elementwise expression node by node: Unary / Binary `forward()`
(include/tannic/tensor.hpp:351-371) and `Function::forward()` (include/tannic/functions.hpp:52-57)
each allocate a temporary and launch one kernel. The change a maintainer would make is four lines:
at the top of each of those bodies,

    #ifdef TANNIC_B200_FUSE
        if (auto fused = ::tannic::b200::try_fused(*this)) return std::move(*fused);
    #endif

plus a forward declaration of `try_fused` and an `#include "fused.hpp"` at the end of functions.hpp.
This script applies exactly that change to COPIES of the two headers, written into the output
directory next to symbolic links to every other header of include/tannic, so that
`-I<output directory>` in place of `-I<reference>/include/tannic` builds the unmodified front-end and
the reference's own tests with whole-expression fusion as the default path. Nothing of the reference
is stored in this repository: the output directory is a build artefact.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

HOOK = """#ifdef TANNIC_B200_FUSE
    if (auto fused_by_default = ::tannic::b200::try_fused(*this)) return std::move(*fused_by_default);
#endif
"""

# tensor.hpp defines the forward() bodies inside `namespace tannic { ... }`, so the declaration opens
# `b200` relative to it; <optional> is included at the top of the file, outside any namespace.
DECLARATION = """#ifdef TANNIC_B200_FUSE
namespace b200 {
// The whole elementwise expression as one kernel, or nothing when it does not fit (defined in fused.hpp).
template <class Expression> std::optional<Tensor> try_fused(Expression const& expression);
}
#endif

"""

TENSOR_ANCHORS = [
    "Tensor expression::Unary<Operation, Operand>::forward(Context const& context) const {",
    "Tensor expression::Binary<Operation, Operand, Cooperand>::forward(Context const& context) const {",
    "Tensor expression::Binary<Operation, Operand, Scalar>::forward(Context const& context) const {",
]
FUNCTION_ANCHOR = "Tensor forward(Context const& context) const {"


def insert_after(text: str, anchor: str, addition: str, what: str) -> str:
    if text.count(anchor) != 1:
        raise SystemExit(f"make_overlay: expected exactly one '{anchor}' in {what}, found {text.count(anchor)}")
    at = text.index(anchor) + len(anchor)
    line_end = text.index("\n", at) + 1
    return text[:line_end] + addition + text[line_end:]


def before_last_endif(text: str, addition: str, what: str) -> str:
    """Inside the include guard: a second inclusion of the header must skip the addition too."""
    at = text.rfind("#endif")
    if at < 0:
        raise SystemExit(f"make_overlay: no include guard found in {what}")
    return text[:at] + addition + text[at:]


def patch_tensor(text: str) -> str:
    first = TENSOR_ANCHORS[0]
    if text.count(first) != 1:
        raise SystemExit("make_overlay: Unary::forward not found in tensor.hpp")
    # the declaration goes in front of the template header line that precedes the first forward body
    body_at = text.index(first)
    template_at = text.rindex("template<", 0, body_at)
    text = text[:template_at] + DECLARATION + text[template_at:]
    for anchor in TENSOR_ANCHORS:
        text = insert_after(text, anchor, HOOK, "tensor.hpp")
    text = "#ifdef TANNIC_B200_FUSE\n#include <optional>\n#endif\n" + text
    return before_last_endif(text, '#ifdef TANNIC_B200_FUSE\n#include "functions.hpp"  // brings fused.hpp with it\n#endif\n', "tensor.hpp")


def patch_functions(text: str) -> str:
    text = insert_after(text, FUNCTION_ANCHOR, HOOK.replace("    if", "        if"), "functions.hpp")
    return before_last_endif(text, '#ifdef TANNIC_B200_FUSE\n#include "fused.hpp"\n#endif\n', "functions.hpp")


def main(reference: str, out: str) -> None:
    source = Path(reference) / "include" / "tannic"
    target = Path(out)
    if not (source / "tensor.hpp").exists():
        raise SystemExit(f"make_overlay: {source} is not the reference's include/tannic")
    target.mkdir(parents=True, exist_ok=True)
    for entry in sorted(source.iterdir()):
        link = target / entry.name
        if link.is_symlink() or link.exists():
            if link.is_dir() and not link.is_symlink():
                raise SystemExit(f"make_overlay: {link} is a real directory")
            link.unlink()
        if entry.name == "tensor.hpp":
            link.write_text(patch_tensor(entry.read_text()))
        elif entry.name == "functions.hpp":
            link.write_text(patch_functions(entry.read_text()))
        else:
            os.symlink(entry.resolve(), link)
    print(f"make_overlay: {target} = {source} with Unary / Binary / Function forward() fused by default")


if __name__ == "__main__":
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    main(sys.argv[1], sys.argv[2])
