// SPIR-V (assembly text form) front end for SPV_ARM_graph modules and the TOSA.001000.1
// extended-instruction registry.
//
// The reference receives binary SPIR-V in vkCreateDataGraphPipelinesARM and lowers it with a
// SPIRV-Tools pass (graph/graph_pass_ext_inst.cpp:25-82) helped by GraphExtInstContext
// (graph/graph_ext_inst_context.cpp) and the per-op decoders of GraphTosa10ExtInst
// (graph/graph_tosa_1_0_ext_inst.cpp).  The numeric opcode tables of SPIR-V and of the TOSA
// instruction set live in SPIRV-Headers, which the reference does not vendor, so this front end
// works on the assembly text — the form of the reference's own tests/shader/*.spvasm fixtures —
// where instructions and TOSA operators appear by name.  The lowering steps and their order are
// the reference's: graph constants, then inputs/outputs, then the graph body in order.
#include <cmath>
#include <cstring>
#include <functional>
#include <map>
#include <sstream>
#include <unordered_map>

#include "graph_pipeline.hpp"

namespace mlel {

namespace {

struct Inst {
    std::string op;
    std::string result;                // without '%', empty if none
    std::vector<std::string> operands; // ids keep their '%', strings keep their quotes
    int line{0};
};

[[noreturn]] void fail(const std::string &msg) { throw std::runtime_error("spvasm: " + msg); }

std::vector<Inst> parseText(const std::string &text) {
    std::vector<Inst> insts;
    std::istringstream stream(text);
    std::string line;
    int lineNo = 0;
    while (std::getline(stream, line)) {
        ++lineNo;
        std::vector<std::string> tokens;
        size_t i = 0;
        while (i < line.size()) {
            const char c = line[i];
            if (c == ';') {
                break; // comment to end of line
            }
            if (c == ' ' || c == '\t' || c == '\r') {
                ++i;
                continue;
            }
            if (c == '"') {
                size_t j = i + 1;
                while (j < line.size() && line[j] != '"') {
                    j += line[j] == '\\' ? 2 : 1;
                }
                tokens.push_back(line.substr(i, j + 1 - i));
                i = j + 1;
                continue;
            }
            size_t j = i;
            while (j < line.size() && line[j] != ' ' && line[j] != '\t' && line[j] != '\r') {
                ++j;
            }
            tokens.push_back(line.substr(i, j - i));
            i = j;
        }
        if (tokens.empty()) {
            continue;
        }
        Inst inst;
        inst.line = lineNo;
        size_t k = 0;
        if (tokens.size() >= 3 && tokens[0][0] == '%' && tokens[1] == "=") {
            inst.result = tokens[0].substr(1);
            k = 2;
        }
        if (k >= tokens.size() || tokens[k].rfind("Op", 0) != 0) {
            fail("line " + std::to_string(lineNo) + ": expected an instruction");
        }
        inst.op = tokens[k];
        inst.operands.assign(tokens.begin() + long(k) + 1, tokens.end());
        insts.push_back(std::move(inst));
    }
    return insts;
}

std::string idOf(const std::string &token) {
    if (token.empty() || token[0] != '%') {
        fail("expected an id, found '" + token + "'");
    }
    return token.substr(1);
}

// Name -> GraphPipeline call for every operator of the TOSA.001000.1 set
// (graph/graph_tosa_1_0_ext_inst.cpp:41-108).  `built` tells whether this build lowers it.
struct TosaEntry {
    const char *name;
    bool built;
};
const TosaEntry kTosaOps[] = {
    {"ABS", true},          {"ADD", true},           {"ARGMAX", true},
    {"ARITHMETIC_RIGHT_SHIFT", true},                {"AVG_POOL2D", true},
    {"BITWISE_AND", true},  {"BITWISE_NOT", true},   {"BITWISE_OR", true},
    {"BITWISE_XOR", true},  {"CAST", true},          {"CEIL", true},
    {"CLAMP", true},        {"CLZ", true},           {"CONCAT", true},
    {"CONV2D", true},       {"CONV3D", true},       {"COS", true},
    {"DEPTHWISE_CONV2D", true},                      {"EQUAL", true},
    {"ERF", true},         {"EXP", true},          {"FFT2D", true},
    {"FLOOR", true},       {"GATHER", true},       {"GREATER", true},
    {"GREATER_EQUAL", true},                         {"INTDIV", true},
    {"LOG", true},         {"LOGICAL_AND", true},   {"LOGICAL_LEFT_SHIFT", true},
    {"LOGICAL_NOT", true},  {"LOGICAL_OR", true},    {"LOGICAL_RIGHT_SHIFT", true},
    {"LOGICAL_XOR", true},  {"MATMUL", true},        {"MAX_POOL2D", true},
    {"MAXIMUM", true},      {"MINIMUM", true},       {"MUL", true},
    {"NEGATE", true},       {"PAD", true},           {"POW", true},
    {"RECIPROCAL", true},  {"REDUCE_ALL", true},    {"REDUCE_ANY", true},
    {"REDUCE_MAX", true},   {"REDUCE_MIN", true},    {"REDUCE_PRODUCT", true},
    {"REDUCE_SUM", true},   {"RESCALE", true},       {"RESHAPE", true},
    {"RESIZE", true},      {"REVERSE", true},      {"RFFT2D", true},
    {"RSQRT", true},       {"SCATTER", true},      {"SELECT", true},
    {"SIGMOID", true},     {"SIN", true},          {"SLICE", true},
    {"SUB", true},          {"TABLE", true},         {"TANH", true},
    {"TILE", true},        {"TRANSPOSE", true},     {"TRANSPOSE_CONV2D", true},
};

const std::unordered_map<std::string, BinaryOp> kBinaryOps = {
    {"ADD", BIN_ADD},
    {"SUB", BIN_SUB},
    {"BITWISE_AND", BIN_BITWISE_AND},
    {"BITWISE_OR", BIN_BITWISE_OR},
    {"BITWISE_XOR", BIN_BITWISE_XOR},
    {"LOGICAL_AND", BIN_LOGICAL_AND},
    {"LOGICAL_OR", BIN_LOGICAL_OR},
    {"LOGICAL_XOR", BIN_LOGICAL_XOR},
    {"LOGICAL_LEFT_SHIFT", BIN_LOGICAL_LEFT_SHIFT},
    {"LOGICAL_RIGHT_SHIFT", BIN_LOGICAL_RIGHT_SHIFT},
    {"INTDIV", BIN_INTDIV},
    {"MAXIMUM", BIN_MAXIMUM},
    {"MINIMUM", BIN_MINIMUM},
    {"EQUAL", BIN_EQUAL},
    {"GREATER", BIN_GREATER},
    {"GREATER_EQUAL", BIN_GREATER_EQUAL},
    {"POW", BIN_POW},
};
const std::unordered_map<std::string, UnaryOp> kUnaryOps = {
    {"ABS", UN_ABS},
    {"BITWISE_NOT", UN_BITWISE_NOT},
    {"CLZ", UN_CLZ},
    {"LOGICAL_NOT", UN_LOGICAL_NOT},
    {"CEIL", UN_CEIL},
    {"COS", UN_COS},
    {"ERF", UN_ERF},
    {"EXP", UN_EXP},
    {"FLOOR", UN_FLOOR},
    {"LOG", UN_LOG},
    {"RECIPROCAL", UN_RECIPROCAL},
    {"RSQRT", UN_RSQRT},
    {"SIGMOID", UN_SIGMOID},
    {"SIN", UN_SIN},
    {"TANH", UN_TANH},
};
const std::unordered_map<std::string, ReduceOp> kReduceOps = {
    {"REDUCE_SUM", RED_SUM},         {"REDUCE_MAX", RED_MAX}, {"REDUCE_MIN", RED_MIN},
    {"REDUCE_PRODUCT", RED_PRODUCT}, {"REDUCE_ALL", RED_ALL}, {"REDUCE_ANY", RED_ANY},
};

// A scalar constant: integers are kept as the sign-extended value of their declared width
// (unsigned SPIR-V integers are reinterpreted as signed of the same width, as
// graph/graph_ext_inst_context.hpp:88-110 does), floats as double.
struct Scalar {
    bool isFloat{false};
    int64_t i{0};
    double f{0.0};
    template <typename T> T as() const { return isFloat ? T(f) : T(i); }
};

class Lowering {
  public:
    Lowering(GraphPipeline &pipeline, std::vector<Inst> insts) : pipeline_(pipeline), insts_(std::move(insts)) {
        for (size_t k = 0; k < insts_.size(); ++k) {
            if (!insts_[k].result.empty()) {
                defs_[insts_[k].result] = k;
            }
            if (insts_[k].op == "OpDecorate" && insts_[k].operands.size() >= 3) {
                const auto id = idOf(insts_[k].operands[0]);
                const auto &what = insts_[k].operands[1];
                const uint64_t value = std::stoull(insts_[k].operands[2]);
                if (what == "DescriptorSet") {
                    sets_[id] = value;
                } else if (what == "Binding") {
                    bindings_[id] = value;
                }
            }
        }
    }

    void run() {
        // graph/graph_layer.cpp:373-395 validateGraphExtInstImports
        for (const auto &inst : insts_) {
            if (inst.op == "OpExtInstImport") {
                const auto name = unquote(inst.operands.at(0));
                if (!extInstSetRegistered(name)) {
                    fail("Unsupported extension " + name);
                }
                imports_[inst.result] = name;
            }
        }
        bool any = false;
        for (size_t k = 0; k < insts_.size(); ++k) {
            if (insts_[k].op == "OpGraphEntryPointARM") {
                any = true;
                handleGraphConstants();
                handleInputsAndOutputs(insts_[k]);
                handleGraph(idOf(insts_[k].operands.at(0)));
            }
        }
        if (!any) {
            fail("module has no OpGraphEntryPointARM");
        }
    }

  private:
    static std::string unquote(const std::string &s) {
        return s.size() >= 2 && s.front() == '"' ? s.substr(1, s.size() - 2) : s;
    }

    const Inst &def(const std::string &id) const {
        const auto it = defs_.find(id);
        if (it == defs_.end()) {
            fail("undefined id %" + id);
        }
        return insts_[it->second];
    }

    // ---- types ----
    struct ElemType {
        int32_t dtype;
        int width;
        bool isFloat;
    };

    ElemType elemType(const std::string &typeId) const {
        const Inst &t = def(typeId);
        if (t.op == "OpTypeInt") {
            const int width = std::stoi(t.operands.at(0));
            switch (width) { // always signed formats: graph/graph_ext_inst_context.cpp:355-370
            case 8:
                return {MLEL_I8, 8, false};
            case 16:
                return {MLEL_I16, 16, false};
            case 32:
                return {MLEL_I32, 32, false};
            case 64:
                return {MLEL_I64, 64, false};
            default:
                fail("Unsupported integer tensor format: width " + std::to_string(width));
            }
        }
        if (t.op == "OpTypeBool") {
            return {MLEL_BOOL, 8, false};
        }
        if (t.op == "OpTypeFloat") {
            const int width = std::stoi(t.operands.at(0));
            const std::string enc = t.operands.size() > 1 ? t.operands[1] : "";
            if (width == 32 && enc.empty()) {
                return {MLEL_F32, 32, true};
            }
            if (width == 16 && enc.empty()) {
                return {MLEL_F16, 16, true};
            }
            if (width == 16 && enc == "BFloat16KHR") {
                return {MLEL_BF16, 16, true};
            }
            throw UnsupportedError("Unsupported float tensor format: width " + std::to_string(width) + " " + enc);
        }
        fail("%" + typeId + " is not a scalar type");
    }

    // Resolves the tensor type behind a type id or behind the result type of a value.
    const Inst &tensorType(const std::string &id) const {
        const Inst *inst = &def(id);
        for (int depth = 0; depth < 8; ++depth) {
            if (inst->op == "OpTypeTensorARM") {
                return *inst;
            }
            if (inst->op == "OpTypeStruct" || inst->op == "OpTypeArray") {
                inst = &def(idOf(inst->operands.at(0)));
            } else if (inst->op == "OpTypePointer") {
                inst = &def(idOf(inst->operands.at(1)));
            } else if (inst->op.rfind("OpType", 0) == 0) {
                break;
            } else {
                inst = &def(idOf(inst->operands.at(0))); // a value: its first operand is its result type
            }
        }
        fail("%" + id + " has no tensor type");
    }

    std::vector<int64_t> tensorShape(const Inst &tt) const {
        if (tt.operands.size() < 3) {
            return {}; // unshaped: takes its shape from the bound resource
        }
        return constVector<int64_t>(idOf(tt.operands[2]));
    }

    size_t tensorElemCount(const Inst &tt) const {
        size_t n = 1;
        for (auto d : tensorShape(tt)) {
            n *= size_t(d);
        }
        return n;
    }

    // ---- constants ----
    Scalar constScalar(const std::string &id) const {
        const Inst &c = def(id);
        Scalar s;
        if (c.op == "OpConstantTrue" || c.op == "OpSpecConstantTrue") {
            s.i = 1;
            return s;
        }
        if (c.op == "OpConstantFalse" || c.op == "OpSpecConstantFalse") {
            s.i = 0;
            return s;
        }
        if (c.op == "OpConstantNull") {
            return s;
        }
        if (c.op != "OpConstant" && c.op != "OpSpecConstant") {
            fail("%" + id + " is not a scalar constant (" + c.op + ")");
        }
        const ElemType et = elemType(idOf(c.operands.at(0)));
        const std::string &lit = c.operands.at(1);
        if (et.isFloat) {
            s.isFloat = true;
            s.f = std::stod(lit);
            return s;
        }
        // Low `width` bits, sign-extended.
        uint64_t bits;
        if (!lit.empty() && lit[0] == '-') {
            bits = uint64_t(std::stoll(lit, nullptr, 0));
        } else {
            bits = std::stoull(lit, nullptr, 0);
        }
        if (et.width < 64) {
            const uint64_t mask = (uint64_t(1) << et.width) - 1;
            bits &= mask;
            if (bits >> (et.width - 1)) {
                bits |= ~mask;
            }
        }
        s.i = int64_t(bits);
        return s;
    }

    bool isCompositeOp(const std::string &op) const {
        return op == "OpConstantComposite" || op == "OpSpecConstantComposite";
    }
    bool isReplicateOp(const std::string &op) const {
        return op == "OpConstantCompositeReplicateEXT" || op == "OpSpecConstantCompositeReplicateEXT";
    }

    void flatten(const std::string &id, std::vector<Scalar> &out) const {
        const Inst &c = def(id);
        if (isCompositeOp(c.op) || isReplicateOp(c.op)) {
            for (size_t k = 1; k < c.operands.size(); ++k) {
                flatten(idOf(c.operands[k]), out);
            }
        } else {
            out.push_back(constScalar(id));
        }
    }

    // graph/graph_ext_inst_context.hpp:192-227 getConstVector
    std::vector<Scalar> constScalars(const std::string &id) const {
        const Inst &c = def(id);
        std::vector<Scalar> values;
        if (isCompositeOp(c.op) || isReplicateOp(c.op)) {
            flatten(id, values);
            if (isReplicateOp(c.op)) {
                const Inst &typeInst = def(idOf(c.operands.at(0)));
                size_t count = values.size();
                if (typeInst.op == "OpTypeTensorARM") {
                    count = tensorElemCount(typeInst);
                } else if (typeInst.op == "OpTypeArray") {
                    count = size_t(constScalar(idOf(typeInst.operands.at(1))).i);
                }
                // tryExpandReplicatedPattern, graph/graph_ext_inst_context.hpp:42-61
                if (values.size() != count) {
                    if (values.empty() || count % values.size() != 0) {
                        fail("Unexpected replicated constant element count for id: " + id);
                    }
                    const auto pattern = values;
                    while (values.size() < count) {
                        values.insert(values.end(), pattern.begin(), pattern.end());
                    }
                }
            }
        } else if (c.op == "OpConstantNull") {
            const Inst &typeInst = def(idOf(c.operands.at(0)));
            if (typeInst.op != "OpTypeTensorARM") {
                fail("OpConstantNull of a non-tensor type used as a vector");
            }
            values.resize(tensorElemCount(typeInst));
        } else {
            fail("Missing declared composite constant for id: " + id);
        }
        return values;
    }

    template <typename T> std::vector<T> constVector(const std::string &id) const {
        std::vector<T> out;
        for (const auto &s : constScalars(id)) {
            out.push_back(s.as<T>());
        }
        return out;
    }

    bool boolConstant(const std::string &id) const {
        const Inst &c = def(id);
        if (c.op == "OpConstantTrue" || c.op == "OpSpecConstantTrue") {
            return true;
        }
        if (c.op == "OpConstantFalse" || c.op == "OpSpecConstantFalse") {
            return false; // spec constants are frozen at their defaults (graph_layer.cpp:94-107)
        }
        fail("Expected boolean constant for id %" + id + ", found " + c.op);
    }

    // ---- tensors ----
    int32_t &slot(const std::string &id, uint32_t arrayIndex) {
        auto &arr = tensorMap_[id];
        if (arr.size() <= arrayIndex) {
            arr.resize(arrayIndex + 1, -1);
        }
        return arr[arrayIndex];
    }

    // graph/graph_ext_inst_context.cpp:309-353 makeCompositeTensor
    int32_t makeCompositeTensor(const std::string &id) {
        const Inst &tt = tensorType(id);
        const ElemType et = elemType(idOf(tt.operands.at(0)));
        const auto dims = tensorShape(tt);
        const auto values = constScalars(id);
        size_t count = 1;
        for (auto d : dims) {
            count *= size_t(d);
        }
        if (values.size() != count) {
            fail("constant %" + id + " has " + std::to_string(values.size()) + " elements, its type " +
                 std::to_string(count));
        }
        std::vector<uint8_t> bytes(count * size_t(elemSize(et.dtype)));
        for (size_t k = 0; k < count; ++k) {
            switch (et.dtype) {
            case MLEL_BOOL:
            case MLEL_I8: {
                const int8_t v = values[k].as<int8_t>();
                std::memcpy(&bytes[k], &v, 1);
                break;
            }
            case MLEL_I16: {
                const int16_t v = values[k].as<int16_t>();
                std::memcpy(&bytes[2 * k], &v, 2);
                break;
            }
            case MLEL_I32: {
                const int32_t v = values[k].as<int32_t>();
                std::memcpy(&bytes[4 * k], &v, 4);
                break;
            }
            case MLEL_I64: {
                const int64_t v = values[k].as<int64_t>();
                std::memcpy(&bytes[8 * k], &v, 8);
                break;
            }
            case MLEL_F32: {
                const float v = values[k].as<float>();
                std::memcpy(&bytes[4 * k], &v, 4);
                break;
            }
            default:
                throw UnsupportedError("Unsupported composite tensor format: " + std::to_string(et.dtype));
            }
        }
        return pipeline_.makeConstCompositeTensor(et.dtype, dims, bytes.data());
    }

    // graph/graph_ext_inst_context.cpp:227-283 getTensor
    int32_t getTensor(const std::string &id, uint32_t arrayIndex = 0) {
        int32_t &cached = slot(id, arrayIndex);
        if (cached >= 0) {
            return cached;
        }
        const Inst &inst = def(id);
        int32_t t = -1;
        if (inst.op == "OpCompositeExtract") {
            return getTensor(idOf(inst.operands.at(1)), uint32_t(std::stoul(inst.operands.at(2))));
        } else if (inst.op == "OpGraphInputARM") {
            fail("OpGraphInputARM tensor requested before graph inputs were connected");
        } else if (isCompositeOp(inst.op) || isReplicateOp(inst.op) || inst.op == "OpConstantNull") {
            t = makeCompositeTensor(id);
        } else if (inst.op == "OpExtInst") {
            // a two-result instruction (FFT2D, RFFT2D) returns a struct: member `arrayIndex` is this tensor's type
            const Inst &resultType = def(idOf(inst.operands.at(0)));
            const bool isStruct = resultType.op == "OpTypeStruct";
            if (isStruct && arrayIndex >= resultType.operands.size()) {
                fail("result %" + id + " has no member " + std::to_string(arrayIndex));
            }
            const Inst &tt = tensorType(isStruct ? idOf(resultType.operands.at(arrayIndex)) : idOf(inst.operands.at(0)));
            const auto dims = tensorShape(tt);
            if (dims.empty()) {
                fail("intermediate tensor %" + id + " has an unshaped type");
            }
            t = pipeline_.makeTensor(elemType(idOf(tt.operands.at(0))).dtype, dims);
        } else if (inst.op == "OpGraphConstantARM") {
            t = pipeline_.getConstTensor(uint32_t(std::stoul(inst.operands.at(1))));
        } else if (inst.op == "OpVariable") {
            const auto s = sets_.find(id);
            if (s == sets_.end()) {
                fail("variable %" + id + " has no DescriptorSet decoration");
            }
            const auto b = bindings_.find(id);
            t = pipeline_.getTensor(uint32_t(s->second), b == bindings_.end() ? 0u : uint32_t(b->second), arrayIndex);
        } else {
            fail("Unsupported instruction type in getTensor: " + inst.op);
        }
        slot(id, arrayIndex) = t;
        return t;
    }

    // getOrMakeCompositeTensor, graph/graph_ext_inst_context.cpp:291-307
    int32_t attributeTensor(const std::string &id) { return getTensor(id, 0); }

    // ---- graph walk ----
    void handleGraphConstants() {
        for (const auto &inst : insts_) {
            if (inst.op == "OpGraphConstantARM" && slot(inst.result, 0) < 0) {
                slot(inst.result, 0) = pipeline_.getConstTensor(uint32_t(std::stoul(inst.operands.at(1))));
            }
        }
    }

    struct GraphBody {
        size_t begin, end; // instruction range (after OpGraphARM, up to OpGraphEndARM)
        size_t numInputs;
    };

    GraphBody body(const std::string &graphId) const {
        const auto it = defs_.find(graphId);
        if (it == defs_.end() || insts_[it->second].op != "OpGraphARM") {
            fail("%" + graphId + " is not an OpGraphARM");
        }
        GraphBody b{it->second + 1, it->second + 1, 0};
        const Inst &gt = def(idOf(insts_[it->second].operands.at(0)));
        if (gt.op != "OpTypeGraphARM") {
            fail("graph type expected");
        }
        b.numInputs = size_t(std::stoul(gt.operands.at(0)));
        while (b.end < insts_.size() && insts_[b.end].op != "OpGraphEndARM") {
            ++b.end;
        }
        return b;
    }

    // graph/graph_ext_inst_context.cpp:77-145
    void handleInputsAndOutputs(const Inst &entry) {
        const GraphBody b = body(idOf(entry.operands.at(0)));
        // OpGraphEntryPointARM <graph id> <name> [interface ids: inputs then outputs]
        std::vector<std::string> iface;
        for (size_t k = 2; k < entry.operands.size(); ++k) {
            iface.push_back(idOf(entry.operands[k]));
        }
        for (size_t k = b.begin; k < b.end; ++k) {
            const Inst &inst = insts_[k];
            if (inst.op == "OpGraphInputARM") {
                const auto inputIndex = size_t(constScalar(idOf(inst.operands.at(1))).i);
                const uint32_t arrayIndex =
                    inst.operands.size() > 2 ? uint32_t(constScalar(idOf(inst.operands[2])).i) : 0u;
                const int32_t t = getTensor(iface.at(inputIndex), arrayIndex);
                pipeline_.makeInput(t);
                slot(inst.result, 0) = t;
            }
        }
        for (size_t k = b.begin; k < b.end; ++k) {
            const Inst &inst = insts_[k];
            if (inst.op != "OpGraphSetOutputARM") {
                continue;
            }
            const std::string valueId = idOf(inst.operands.at(0));
            const auto outputIndex = size_t(constScalar(idOf(inst.operands.at(1))).i);
            const uint32_t arrayIndex = inst.operands.size() > 2 ? uint32_t(constScalar(idOf(inst.operands[2])).i) : 0u;
            const int32_t outTensor = getTensor(iface.at(b.numInputs + outputIndex), arrayIndex);
            pipeline_.makeOutput(outTensor);
            const Inst &value = def(valueId);
            if (isCompositeOp(value.op) || isReplicateOp(value.op) || value.op == "OpGraphInputARM" ||
                value.op == "OpGraphConstantARM") {
                // pass-through outputs are lowered to CAST (graph_ext_inst_context.cpp:122-129)
                pipeline_.makeCast(getTensor(valueId), outTensor, "CAST");
            } else if (value.op == "OpCompositeExtract") {
                slot(idOf(value.operands.at(1)), uint32_t(std::stoul(value.operands.at(2)))) = outTensor;
            } else {
                slot(valueId, 0) = outTensor;
            }
        }
    }

    // graph/graph_pass_ext_inst.cpp:46-82
    void handleGraph(const std::string &graphId) {
        const GraphBody b = body(graphId);
        for (size_t k = b.begin; k < b.end; ++k) {
            const Inst &inst = insts_[k];
            if (inst.op == "OpExtInst") {
                const auto set = imports_.find(idOf(inst.operands.at(1)));
                if (set == imports_.end()) {
                    fail("Invalid extended instruction-set import id " + inst.operands.at(1));
                }
                if (set->second != "TOSA.001000.1") {
                    throw UnsupportedError("Unsupported extension " + set->second);
                }
                handleTosa(inst);
            } else if (inst.op == "OpCompositeExtract" || inst.op == "OpGraphInputARM" ||
                       inst.op == "OpGraphSetOutputARM") {
                continue;
            } else {
                fail("Unsupported graph instruction " + inst.op);
            }
        }
    }

    // One decoder per operator; operand order as documented in graph/graph_tosa_1_0_ext_inst.cpp:315-1032.
    void handleTosa(const Inst &inst) {
        const std::string &name = inst.operands.at(2);
        std::vector<std::string> a; // argument ids after (type, set, opcode)
        for (size_t k = 3; k < inst.operands.size(); ++k) {
            a.push_back(idOf(inst.operands[k]));
        }
        const auto argc = [&](size_t n) {
            if (a.size() != n) {
                fail(name + " expects " + std::to_string(n) + " operands, found " + std::to_string(a.size()));
            }
        };
        const auto result = [&]() { return getTensor(inst.result); };
        auto &p = pipeline_;

        if (name == "CONV2D" || name == "DEPTHWISE_CONV2D") {
            // pad stride dilation accType localBound input weight bias inputZeroPoint weightZeroPoint
            argc(10);
            const auto pad = constVector<int32_t>(a[0]), stride = constVector<int32_t>(a[1]),
                       dilation = constVector<int32_t>(a[2]);
            const auto accType = constScalar(a[3]).as<uint32_t>();
            (void)boolConstant(a[4]); // local_bound is decoded and ignored
            const auto inZp = constVector<int8_t>(a[8]), wZp = constVector<int8_t>(a[9]);
            if (name == "CONV2D") {
                p.makeConv2D(getTensor(a[5]), result(), getTensor(a[6]), getTensor(a[7]), pad, stride, dilation,
                             inZp.at(0), wZp.at(0), accType, name);
            } else {
                p.makeDepthwiseConv2D(getTensor(a[5]), result(), getTensor(a[6]), getTensor(a[7]), pad, stride,
                                      dilation, inZp.at(0), wZp.at(0), accType, name);
            }
        } else if (name == "MATMUL") {
            argc(4); // input1 input2 input1ZeroPoint input2ZeroPoint
            p.makeMatmul(getTensor(a[0]), getTensor(a[1]), result(), constVector<int8_t>(a[2]).at(0),
                         constVector<int8_t>(a[3]).at(0), name);
        } else if (name == "RESCALE") {
            // scale32 roundingMode perChannel inputUnsigned outputUnsigned input multiplier shift inZp outZp
            argc(10);
            const bool scale32 = boolConstant(a[0]);
            const auto roundingMode = constScalar(a[1]).as<uint32_t>(); // 1 single, 2 inexact, 3 double
            const bool perChannel = boolConstant(a[2]), inU = boolConstant(a[3]), outU = boolConstant(a[4]);
            const int32_t mult = attributeTensor(a[6]), shift = attributeTensor(a[7]);
            p.makeRescale(getTensor(a[5]), result(), constVector<int32_t>(a[8]).at(0),
                          constVector<int32_t>(a[9]).at(0), mult, shift, scale32, roundingMode == 3, perChannel, inU,
                          outU, name);
        } else if (name == "AVG_POOL2D") {
            argc(7); // kernel stride pad accType input inputZeroPoint outputZeroPoint
            p.makeAvgPool2D(getTensor(a[4]), result(), constVector<int32_t>(a[0]), constVector<int32_t>(a[1]),
                            constVector<int32_t>(a[2]), constScalar(a[3]).as<uint32_t>(),
                            constVector<int8_t>(a[5]).at(0), constVector<int8_t>(a[6]).at(0), name);
        } else if (name == "MAX_POOL2D") {
            argc(5); // kernel stride pad nanMode input
            p.makeMaxPool2D(getTensor(a[4]), result(), constVector<int32_t>(a[0]), constVector<int32_t>(a[1]),
                            constVector<int32_t>(a[2]), constScalar(a[3]).as<uint32_t>(), name);
        } else if (name == "TABLE") {
            argc(2); // input table
            p.makeTable(getTensor(a[0]), result(), attributeTensor(a[1]), name);
        } else if (name == "TRANSPOSE") {
            argc(2); // perms input
            p.makeTranspose(getTensor(a[1]), result(), constVector<uint32_t>(a[0]), name);
        } else if (name == "CONCAT") {
            if (a.size() < 2) {
                fail("CONCAT expects an axis and at least one input");
            }
            std::vector<int32_t> inputs;
            for (size_t k = 1; k < a.size(); ++k) {
                inputs.push_back(getTensor(a[k]));
            }
            p.makeConcat(inputs, result(), constScalar(a[0]).as<uint32_t>(), name);
        } else if (name == "CLAMP") {
            argc(4); // minVal maxVal nanMode input
            p.makeClamp(getTensor(a[3]), result(), constScalar(a[0]).as<double>(), constScalar(a[1]).as<double>(),
                        constScalar(a[2]).as<uint32_t>(), name);
        } else if (name == "MAXIMUM" || name == "MINIMUM") {
            argc(3); // nanMode input1 input2
            p.makeBinary(kBinaryOps.at(name), getTensor(a[1]), getTensor(a[2]), result(),
                         constScalar(a[0]).as<uint32_t>(), name);
        } else if (kBinaryOps.count(name)) {
            argc(2); // input1 input2
            p.makeBinary(kBinaryOps.at(name), getTensor(a[0]), getTensor(a[1]), result(), 1, name);
        } else if (kUnaryOps.count(name)) {
            argc(1);
            p.makeUnary(kUnaryOps.at(name), getTensor(a[0]), result(), name);
        } else if (name == "MUL") {
            argc(3); // input1 input2 shift
            p.makeMul(getTensor(a[0]), getTensor(a[1]), result(), constVector<uint8_t>(a[2]).at(0), name);
        } else if (name == "REDUCE_MAX" || name == "REDUCE_MIN") {
            argc(3); // axis nanMode input
            p.makeReduce(kReduceOps.at(name), getTensor(a[2]), result(), constScalar(a[0]).as<uint32_t>(),
                         constScalar(a[1]).as<uint32_t>(), name);
        } else if (kReduceOps.count(name)) {
            argc(2); // axis input
            p.makeReduce(kReduceOps.at(name), getTensor(a[1]), result(), constScalar(a[0]).as<uint32_t>(), 1, name);
        } else if (name == "CAST") {
            argc(1);
            p.makeCast(getTensor(a[0]), result(), name);
        } else if (name == "RESHAPE") {
            argc(2); // input shape (the output tensor's own shape is what is used)
            (void)constVector<uint32_t>(a[1]);
            p.makeReshape(getTensor(a[0]), result(), name);
        } else if (name == "SLICE") {
            argc(3); // input start size (size is decoded and ignored)
            (void)constVector<uint32_t>(a[2]);
            p.makeSlice(getTensor(a[0]), result(), constVector<uint32_t>(a[1]), name);
        } else if (name == "PAD") {
            argc(3); // input padding padConst
            const int32_t out = result();
            double padConst = 0.0;
            int32_t padConstInt = 0;
            if (p.tensor(out).dtype == MLEL_I32) {
                padConstInt = constVector<int32_t>(a[2]).at(0);
                padConst = double(padConstInt);
            } else {
                padConst = constVector<double>(a[2]).at(0);
                padConstInt = int32_t(padConst);
            }
            p.makePad(getTensor(a[0]), out, attributeTensor(a[1]), padConst, padConstInt, name);
        } else if (name == "ARITHMETIC_RIGHT_SHIFT") {
            argc(3); // round input1 input2
            p.makeArithmeticRightShift(getTensor(a[1]), getTensor(a[2]), result(), boolConstant(a[0]), name);
        } else if (name == "NEGATE") {
            argc(3); // input inputZeroPoint outputZeroPoint
            p.makeNegate(getTensor(a[0]), result(), constVector<int32_t>(a[1]).at(0),
                         constVector<int32_t>(a[2]).at(0), name);
        } else if (name == "SELECT") {
            argc(3);
            p.makeSelect(getTensor(a[0]), getTensor(a[1]), getTensor(a[2]), result(), name);
        } else if (name == "FFT2D") {
            argc(4); // inverse localBound inputReal inputImag
            (void)boolConstant(a[1]);
            p.makeFft2D(getTensor(a[2]), getTensor(a[3]), getTensor(inst.result, 0), getTensor(inst.result, 1),
                        boolConstant(a[0]), name);
        } else if (name == "RFFT2D") {
            argc(2); // localBound input
            (void)boolConstant(a[0]);
            p.makeRfft2D(getTensor(a[1]), getTensor(inst.result, 0), getTensor(inst.result, 1), name);
        } else if (name == "ARGMAX") {
            argc(3); // axis nanMode input
            p.makeArgmax(getTensor(a[2]), result(), constScalar(a[0]).as<uint32_t>(),
                         constScalar(a[1]).as<uint32_t>(), name);
        } else if (name == "GATHER") {
            argc(2); // values indices
            p.makeGather(getTensor(a[0]), getTensor(a[1]), result(), name);
        } else if (name == "SCATTER") {
            argc(3); // valuesIn indices input
            p.makeScatter(getTensor(a[2]), getTensor(a[0]), getTensor(a[1]), result(), name);
        } else if (name == "REVERSE") {
            argc(2); // axis input
            p.makeReverse(getTensor(a[1]), result(), constScalar(a[0]).as<uint32_t>(), name);
        } else if (name == "TILE") {
            argc(2); // input multiples (decoded; the output tensor's shape is what is used)
            (void)constVector<uint32_t>(a[1]);
            p.makeTile(getTensor(a[0]), result(), name);
        } else if (name == "RESIZE") {
            argc(5); // mode input scale offset border
            p.makeResize(getTensor(a[1]), result(), constVector<int32_t>(a[2]), constVector<int32_t>(a[3]),
                         constVector<int32_t>(a[4]), constScalar(a[0]).as<uint32_t>(), name);
        } else if (name == "TRANSPOSE_CONV2D") {
            // outPad stride accType localBound input weight bias inputZeroPoint weightZeroPoint
            argc(9);
            (void)boolConstant(a[3]);
            p.makeTransposeConv2D(getTensor(a[4]), result(), getTensor(a[5]), getTensor(a[6]),
                                  constVector<int32_t>(a[0]), constVector<int32_t>(a[1]),
                                  constVector<int8_t>(a[7]).at(0), constVector<int8_t>(a[8]).at(0),
                                  constScalar(a[2]).as<uint32_t>(), name);
        } else if (name == "CONV3D") {
            // pad stride dilation accType localBound input weight bias inputZeroPoint weightZeroPoint
            argc(10);
            (void)boolConstant(a[4]);
            p.makeConv3D(getTensor(a[5]), result(), getTensor(a[6]), getTensor(a[7]), constVector<int32_t>(a[0]),
                         constVector<int32_t>(a[1]), constVector<int32_t>(a[2]), constVector<int8_t>(a[8]).at(0),
                         constVector<int8_t>(a[9]).at(0), constScalar(a[3]).as<uint32_t>(), name);
        } else {
            bool known = false;
            for (const auto &e : kTosaOps) {
                known |= name == e.name;
            }
            if (known) {
                throw UnsupportedError("TOSA operator " + name + " is not built in this implementation");
            }
            fail("unknown TOSA.001000.1 instruction " + name);
        }
    }

    GraphPipeline &pipeline_;
    std::vector<Inst> insts_;
    std::unordered_map<std::string, size_t> defs_;
    std::unordered_map<std::string, uint64_t> sets_, bindings_;
    std::unordered_map<std::string, std::string> imports_;
    std::unordered_map<std::string, std::vector<int32_t>> tensorMap_;
};

} // namespace

// graph/graph_ext_inst_registry.cpp:36-51: "TOSA.001000.1" and "Arm.MotionEngine.100" are the
// registered sets of the reference; only the TOSA set is on this path.
bool extInstSetRegistered(const std::string &importName) { return importName == "TOSA.001000.1"; }

const std::vector<std::string> &tosaOpNames() {
    static const std::vector<std::string> names = [] {
        std::vector<std::string> v;
        for (const auto &e : kTosaOps) {
            v.emplace_back(e.name);
        }
        return v;
    }();
    return names;
}

bool tosaOpSupported(const std::string &name) {
    for (const auto &e : kTosaOps) {
        if (name == e.name) {
            return e.built;
        }
    }
    return false;
}

void lowerSpvasm(GraphPipeline &pipeline, const std::string &text) {
    Lowering lowering(pipeline, parseText(text));
    lowering.run();
}

} // namespace mlel
