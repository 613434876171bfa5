// One kernel per elementwise expression, for the reference's own expression templates.
//
// The reference evaluates `log(X) + Y * Y - exp(X)` node by node: every Binary / Unary / Function
// `forward()` allocates a full-size temporary and launches one kernel (include/tannic/tensor.hpp:351-371,
// include/tannic/functions.hpp:52-57). `tannic::b200::fused(expression)` walks the same template tree at
// compile time, lists its tensors and nodes, and hands the whole tree to `tn_eltwise_program`, which
// reads every operand once and writes the result once. Anything the program format cannot hold (more
// than TN_PROGRAM_MAX_INPUTS tensors or TN_PROGRAM_MAX_NODES nodes, mixed dtypes, host tensors,
// non-elementwise sub-expressions) falls back to the expression's own `forward()`.
//
// Compiled against the reference's headers (operations.hpp, functions.hpp, callback.hpp); needs no
// change to them. Results equal the node-by-node evaluation: the fused kernel rounds every node to
// the storage dtype.
//
// `try_fused(expression)` is the same walk as an optional: it returns nothing when the tree does not
// fit, so it can be the first statement of the front-end's own forward() bodies (the four-line change
// make_overlay.py applies to copies of tensor.hpp / functions.hpp under -DTANNIC_B200_FUSE), which
// makes one-kernel evaluation the default for `Tensor Z = log(X) + Y * Y - exp(X);`.
#pragma once

#include <optional>
#include <stdexcept>
#include <tuple>
#include <type_traits>
#include <variant>

#include "callback.hpp"
#include "context.hpp"
#include "functions.hpp"
#include "operations.hpp"
#include "tensor.hpp"

#include "tannic_b200.h"

namespace tannic::b200 {

struct Plan {
    const Tensor* inputs[TN_PROGRAM_MAX_INPUTS] = {};
    int n_inputs = 0;
    tn_eltwise_node_t nodes[TN_PROGRAM_MAX_NODES] = {};
    int n_nodes = 0;
    bool ok = true;

    int input(Tensor const& t) {
        for (int i = 0; i < n_inputs; ++i)
            if (inputs[i]->id() == t.id()) return i;  // the same tensor named twice is read once
        if (n_inputs == TN_PROGRAM_MAX_INPUTS) {
            ok = false;
            return 0;
        }
        inputs[n_inputs] = &t;
        return n_inputs++;
    }
    int node(int opcode, int lhs, int rhs, float imm = 0.0f) {
        if (opcode < 0 || n_nodes == TN_PROGRAM_MAX_NODES) {
            ok = false;
            return 0;
        }
        nodes[n_nodes] = tn_eltwise_node_t{static_cast<uint8_t>(opcode), static_cast<uint8_t>(lhs), static_cast<uint8_t>(rhs), imm};
        return TN_PROGRAM_MAX_INPUTS + n_nodes++;
    }
};

template <class Operation> struct opcode_of { static constexpr int value = -1; };
template <> struct opcode_of<operation::Addition> { static constexpr int value = TN_OP_ADD; };
template <> struct opcode_of<operation::Subtraction> { static constexpr int value = TN_OP_SUB; };
template <> struct opcode_of<operation::Multiplication> { static constexpr int value = TN_OP_MUL; };
template <> struct opcode_of<operation::Exponentiation> { static constexpr int value = TN_OP_POW; };
template <> struct opcode_of<operation::Negation> { static constexpr int value = TN_OP_NEG; };
template <> struct opcode_of<function::Log> { static constexpr int value = TN_OP_LOG; };
template <> struct opcode_of<function::Exp> { static constexpr int value = TN_OP_EXP; };
template <> struct opcode_of<function::Sqrt> { static constexpr int value = TN_OP_SQRT; };
template <> struct opcode_of<function::Rsqrt> { static constexpr int value = TN_OP_RSQRT; };
template <> struct opcode_of<function::Abs> { static constexpr int value = TN_OP_ABS; };
template <> struct opcode_of<function::Sin> { static constexpr int value = TN_OP_SIN; };
template <> struct opcode_of<function::Cos> { static constexpr int value = TN_OP_COS; };
template <> struct opcode_of<function::Tan> { static constexpr int value = TN_OP_TAN; };
template <> struct opcode_of<function::Sinh> { static constexpr int value = TN_OP_SINH; };
template <> struct opcode_of<function::Cosh> { static constexpr int value = TN_OP_COSH; };
template <> struct opcode_of<function::Tanh> { static constexpr int value = TN_OP_TANH; };

inline float scalar_as_float(Scalar const& s) {
    switch (s.dtype()) {
        case int8: return static_cast<float>(s.get<int8_t>());
        case int16: return static_cast<float>(s.get<int16_t>());
        case int32: return static_cast<float>(s.get<int32_t>());
        case int64: return static_cast<float>(s.get<int64_t>());
        case float16: return static_cast<float>(s.get<float16_t>());
        case bfloat16: return static_cast<float>(s.get<bfloat16_t>());
        case float32: return s.get<float>();
        case float64: return static_cast<float>(s.get<double>());
        default: throw std::runtime_error("scalar dtype has no elementwise program form");
    }
}

// value id of a sub-expression: tensors are inputs, operators append a node. The last overload
// marks everything else (views, matmul, reductions, ...) as not fusible.
inline int emit(Plan& p, Tensor const& t) { return p.input(t); }

template <class E> int emit(Plan& p, E const&);

template <class Operation, class Operand>
int emit(Plan& p, expression::Unary<Operation, Operand> const& e) {
    const int a = emit(p, std::get<0>(e.operands));
    return p.node(opcode_of<Operation>::value, a, a);
}
template <class Operation, class Operand, class Cooperand>
int emit(Plan& p, expression::Binary<Operation, Operand, Cooperand> const& e) {
    const int a = emit(p, std::get<0>(e.operands));
    if constexpr (std::is_same_v<std::decay_t<Cooperand>, Scalar>) {
        if constexpr (!std::is_same_v<Operation, operation::Multiplication>) {
            p.ok = false;
            return 0;
        } else {
            return p.node(TN_OP_SCALE, a, a, scalar_as_float(std::get<1>(e.operands)));
        }
    } else {
        const int b = emit(p, std::get<1>(e.operands));
        return p.node(opcode_of<Operation>::value, a, b);
    }
}
template <class Functor, class Argument>
int emit(Plan& p, expression::Function<Functor, Argument> const& e) {
    const int a = emit(p, std::get<0>(e.operands));
    float imm = 0.0f;
    if constexpr (std::is_same_v<Functor, function::Rsqrt>) imm = e.operation.epsilon;
    return p.node(opcode_of<Functor>::value, a, a, imm);
}
template <class E>
int emit(Plan& p, E const&) {
    p.ok = false;
    return 0;
}

// The expression as one kernel, or nothing when it does not fit the program format: fewer than
// `min_nodes` nodes (a single node gains nothing and keeps the front-end's own dtype rules), tensors
// that are uninitialised, on the host, strided, of different dtypes or on different devices, a result
// dtype other than the operands'.
template <class E>
std::optional<Tensor> try_fused_with(E const& e, int min_nodes) {
    Plan p;
    emit(p, e);
    if (!p.ok || p.n_nodes < min_nodes || p.n_inputs == 0) return std::nullopt;
    int device_id = -1;
    for (int i = 0; i < p.n_inputs; ++i) {
        Tensor const& t = *p.inputs[i];
        if (!t.is_initialized() || !t.is_contiguous() || !std::holds_alternative<Device>(t.environment()) || t.dtype() != p.inputs[0]->dtype())
            return std::nullopt;
        const int id = std::get<Device>(t.environment()).id();
        if (device_id >= 0 && id != device_id) return std::nullopt;
        device_id = id;
    }
    if (e.dtype() != p.inputs[0]->dtype()) return std::nullopt;
    Tensor result(e.dtype(), e.shape());
    result.initialize(Device(device_id));
    const tn_tensor_t* in[TN_PROGRAM_MAX_INPUTS] = {};
    for (int i = 0; i < p.n_inputs; ++i) in[i] = reinterpret_cast<const tn_tensor_t*>(get_tensor(p.inputs[i]->id()));
    device_t dvc{device_id};
    stream_t stream = pop_stream(&dvc);
    const tn_status st = tn_eltwise_program(in, p.n_inputs, p.nodes, p.n_nodes, reinterpret_cast<tn_tensor_t*>(get_tensor(result.id())),
                                            tn_stream_t{stream.address});
    put_stream(&dvc, stream);
    if (st != TN_SUCCESS) throw std::runtime_error(tn_last_error());
    return result;
}

// The hook of the fused-by-default overlay: trees of two or more nodes.
template <class E>
std::optional<Tensor> try_fused(E const& e) {
    return try_fused_with(e, 2);
}

// The expression evaluated as one kernel (or by its own forward() when it does not fit).
template <class E>
Tensor fused(E const& e) {
    if (auto result = try_fused_with(e, 1)) return std::move(*result);
    return e.forward(Context{});
}

}  // namespace tannic::b200
