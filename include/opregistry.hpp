// Operator registry: shared operator instances keyed by (C++ class, operator kind, name).
// Same mechanics as include/opregistry.hpp:9-71 of the reference (singleton, typeid name of
// the concrete class as the first key, REGISTER_OPERATOR macro), plus a mutex, which the
// reference's registry lacks.
#pragma once

#include <iostream>
#include <mutex>
#include <stdexcept>
#include <typeinfo>
#include <unordered_map>

#include "operator.hpp"

namespace infer {

class OperatorRegistry {
public:
    static OperatorRegistry& getInstance() {
        static OperatorRegistry instance;
        return instance;
    }
    OperatorRegistry(const OperatorRegistry&) = delete;
    OperatorRegistry& operator=(const OperatorRegistry&) = delete;

    void registerOperator(OperatorType type, const std::string& name, std::shared_ptr<Operator> op) {
        if (!op) throw std::invalid_argument("registerOperator: null operator");
        std::lock_guard<std::mutex> lock(mutex_);
        registry_[typeid(*op).name()][static_cast<int>(type)][name] = std::move(op);
    }

    template <typename T, template <typename> class OpClass>
    std::shared_ptr<OpClass<T>> getOperator(OperatorType type, const std::string& name) {
        std::lock_guard<std::mutex> lock(mutex_);
        auto by_class = registry_.find(typeid(OpClass<T>).name());
        if (by_class == registry_.end()) return nullptr;
        auto by_type = by_class->second.find(static_cast<int>(type));
        if (by_type == by_class->second.end()) return nullptr;
        auto by_name = by_type->second.find(name);
        if (by_name == by_type->second.end()) return nullptr;
        return std::dynamic_pointer_cast<OpClass<T>>(by_name->second);
    }

    size_t size() const {
        std::lock_guard<std::mutex> lock(mutex_);
        size_t n = 0;
        for (const auto& c : registry_)
            for (const auto& t : c.second) n += t.second.size();
        return n;
    }

    void listRegisteredOperators(std::ostream& os = std::cout) const {
        std::lock_guard<std::mutex> lock(mutex_);
        os << "=== Registered Operators ===" << std::endl;
        for (const auto& c : registry_) {
            os << "TypeName: " << c.first << std::endl;
            for (const auto& t : c.second) {
                os << "  OperatorType: " << t.first << std::endl;
                for (const auto& n : t.second) os << "    Name: " << n.first << std::endl;
            }
        }
    }

private:
    OperatorRegistry() = default;
    mutable std::mutex mutex_;
    std::unordered_map<std::string, std::unordered_map<int, std::unordered_map<std::string, std::shared_ptr<Operator>>>>
        registry_;
};

// REGISTER_OPERATOR(type, name, classname, data_type): registers one shared instance of
// classname<data_type> under #name.  Re-registration replaces the instance.
#define REGISTER_OPERATOR(type, name, classname, data_type) \
    infer::OperatorRegistry::getInstance().registerOperator(type, #name, std::make_shared<classname<data_type>>())

}  // namespace infer
