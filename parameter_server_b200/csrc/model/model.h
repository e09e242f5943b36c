// Model metadata objects kept on the master so that predictors can find the tables of a trained model.
//
// Parity: pico-ps/model/Model.{h,cpp}: TABLE_INIT_METHOD, OperatorObject, TableObject, ModelStatus, the
// recursive ModelObject (sub-models + tables) and their JSON round trip; all_tables / all_operators
// flatten the tree. SyncHandler resolves (model_name, table_name, op_key) through these objects
// (pico-ps/handler/SyncHandler.h:76-110).
#pragma once
#include <string>
#include <vector>

#include "../common/json.h"
#include "../service/master.h"

namespace psb {

enum class TableInitMethod : int { REMOTE_PS = 0, LOCAL_PS = 1, NON_PS = 2 };
enum class ModelStatus : int { NORMAL = 0, RESTORING = 1, CREATING = 2, DELETING = 3, UPDATING = 4 };

struct OperatorObject {
    std::string key, lib_name, op_name, config_str;
    int32_t handler_id = -1;
    Json to_json() const {
        Json j = Json::object();
        j["key"] = key; j["lib_name"] = lib_name; j["op_name"] = op_name; j["config_str"] = config_str; j["handler_id"] = handler_id;
        return j;
    }
    static OperatorObject from_json(const Json& j) {
        OperatorObject o;
        o.key = j.at("key").as_string(); o.lib_name = j.at("lib_name").as_string(); o.op_name = j.at("op_name").as_string();
        o.config_str = j.at("config_str").as_string(); o.handler_id = (int32_t)j.at("handler_id").as_int(-1);
        return o;
    }
};

struct TableObject {
    std::string table_name, table_uri, lib_name;
    TableInitMethod init_method = TableInitMethod::REMOTE_PS;
    int32_t shard_num = 0, replica_num = 1, storage_id = -1;
    OperatorObject storage_op;
    std::vector<OperatorObject> ops;
    Json to_json() const {
        Json j = Json::object();
        j["table_name"] = table_name; j["table_uri"] = table_uri; j["lib_name"] = lib_name; j["init_method"] = (int)init_method;
        j["shard_num"] = shard_num; j["replica_num"] = replica_num; j["storage_id"] = storage_id; j["storage_op"] = storage_op.to_json();
        Json a = Json::array();
        for (auto& o : ops) a.push_back(o.to_json());
        j["ops"] = a;
        return j;
    }
    static TableObject from_json(const Json& j) {
        TableObject t;
        t.table_name = j.at("table_name").as_string(); t.table_uri = j.at("table_uri").as_string(); t.lib_name = j.at("lib_name").as_string();
        t.init_method = (TableInitMethod)j.at("init_method").as_int(); t.shard_num = (int32_t)j.at("shard_num").as_int();
        t.replica_num = (int32_t)j.at("replica_num").as_int(1); t.storage_id = (int32_t)j.at("storage_id").as_int(-1);
        t.storage_op = OperatorObject::from_json(j.at("storage_op"));
        for (auto& o : j.at("ops").elements()) t.ops.push_back(OperatorObject::from_json(o));
        return t;
    }
    const OperatorObject* find_op(const std::string& key) const {
        for (auto& o : ops) if (o.key == key) return &o;
        return nullptr;
    }
};

struct ModelObject {
    std::string name, type, version;
    ModelStatus status = ModelStatus::NORMAL;
    std::vector<ModelObject> submodels;
    std::vector<TableObject> tables;
    Json to_json() const {
        Json j = Json::object();
        j["name"] = name; j["type"] = type; j["version"] = version; j["status"] = (int)status;
        Json s = Json::array(), t = Json::array();
        for (auto& m : submodels) s.push_back(m.to_json());
        for (auto& tb : tables) t.push_back(tb.to_json());
        j["submodels"] = s; j["tables"] = t;
        return j;
    }
    static ModelObject from_json(const Json& j) {
        ModelObject m;
        m.name = j.at("name").as_string(); m.type = j.at("type").as_string(); m.version = j.at("version").as_string();
        m.status = (ModelStatus)j.at("status").as_int();
        for (auto& s : j.at("submodels").elements()) m.submodels.push_back(from_json(s));
        for (auto& t : j.at("tables").elements()) m.tables.push_back(TableObject::from_json(t));
        return m;
    }
    void all_tables(std::vector<const TableObject*>* out) const {
        for (auto& t : tables) out->push_back(&t);
        for (auto& m : submodels) m.all_tables(out);
    }
    void all_operators(std::vector<const OperatorObject*>* out) const {
        std::vector<const TableObject*> ts;
        all_tables(&ts);
        for (auto* t : ts) for (auto& o : t->ops) out->push_back(&o);
    }
    const TableObject* find_table(const std::string& table_name) const {
        std::vector<const TableObject*> ts;
        all_tables(&ts);
        for (auto* t : ts) if (t->table_name == table_name) return t;
        return nullptr;
    }
};

inline Status set_model(MasterClient& m, const ModelObject& model) { return m.tree_node_set("model/" + model.name, model.to_json().dump()); }
inline Status get_model(MasterClient& m, const std::string& name, ModelObject* out) {
    std::string s;
    PSB_RETURN_IF_ERROR(m.tree_node_get("model/" + name, &s));
    Json j;
    if (!Json::parse(s, &j)) return Status::Error("model JSON does not parse");
    *out = ModelObject::from_json(j);
    return Status::Ok();
}
inline Status delete_model(MasterClient& m, const std::string& name) { return m.tree_node_del("model/" + name); }

}  // namespace psb
